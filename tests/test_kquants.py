"""K-quant super-blocks (Q2K, Q3K, Q4K, Q5K, Q6K, Q8K: candle-core/src/quantized/k_quants.rs:698-1883).

CPU part: the oracle's writers and decoders reproduce the values candle's own tests pin
(candle-core/tests/quantized_tests.rs:437-716).  GPU part: the kernels' decode of seeded random
blocks and of those test vectors against the oracle, bit for bit, for whole-buffer decode, row
lookup and lookup + RMS norm."""
import numpy as np
import pytest
import torch

import oracle
from helpers import bits, from_oracle, ids_tensor, make_kq_blocks, randn, to_oracle

KQ = ["q2k", "q3k", "q4k", "q5k", "q6k", "q8k"]


def ramp_vector(bound, size):
    v = np.arange(size, dtype=np.float32)
    half = np.float32(size) / np.float32(2)
    return (((v - half) * np.float32(bound)).astype(np.float32) / half).astype(np.float32)


def round3(x):
    t = (np.float32(1000.0) * np.asarray(x, np.float32)).astype(np.float32)
    r = np.where(t >= 0, np.floor(t + np.float32(0.5)), np.ceil(t - np.float32(0.5))).astype(np.float32)
    return (r / np.float32(1000.0)).astype(np.float32)


@pytest.mark.parametrize("qtype", KQ)
def test_oracle_reproduces_candles_round_trip_vectors(kats, qtype):
    k = kats[f"quantize_{qtype}"]
    src = ramp_vector(k["bound"], k["size"])
    pts = k["points"]
    assert np.array_equal(src[pts], np.asarray([float(v) for v in k["src_points"]], np.float32))
    dst = oracle.dequantize(oracle.quantize(src, qtype), qtype)
    assert np.abs(dst - src).max() < k["max_abs_error"]
    want = np.asarray([float(v) for v in k["dequantized_points_rounded_3"]], np.float32)
    assert np.array_equal(round3(dst[pts]), want), (round3(dst[pts]), want)  # -0.0 == 0.0, as in assert_eq! on f32
    big = ramp_vector(k["big_bound"], k["size"])
    dst_big = oracle.dequantize(oracle.quantize(big, qtype), qtype)
    assert np.abs(dst_big - big).max() < k["big_max_abs_error"]
    # the cosine vector of the ggml unit tests: RMSE bound (f32 cos of the platform's libm)
    i = np.arange(k["ggml_size"], dtype=np.float32)
    g = (np.float32(0.1) + np.float32(2.0) * np.cos(i).astype(np.float32)).astype(np.float32)
    dg = oracle.dequantize(oracle.quantize(g, qtype), qtype)
    rmse = np.sqrt(np.sum((g - dg).astype(np.float32) ** 2, dtype=np.float32)) / np.float32(g.size)
    assert rmse <= k["ggml_max_rmse"]


@pytest.mark.parametrize("qtype", KQ)
def test_oracle_decoders_against_numpy_statement(qtype):
    """An independent (vectorised numpy) statement of each to_float, on random blocks."""
    rng = np.random.default_rng(7)
    raw = make_kq_blocks(rng, qtype, 40)
    got = oracle.dequantize(raw.reshape(-1), qtype).reshape(40, 256)
    f16 = lambda b: b.copy().view(np.float16).astype(np.float32).reshape(-1)  # noqa: E731
    F = np.float32
    out = np.zeros((40, 256), np.float32)

    def scale_min_k4(sc):
        d = np.zeros((40, 8), np.uint8)
        m = np.zeros((40, 8), np.uint8)
        d[:, :4], m[:, :4] = sc[:, 0:4] & 63, sc[:, 4:8] & 63
        d[:, 4:] = (sc[:, 8:12] & 0xF) | ((sc[:, 0:4] >> 6) << 4)
        m[:, 4:] = (sc[:, 8:12] >> 4) | ((sc[:, 4:8] >> 6) << 4)
        return d.astype(F), m.astype(F)

    if qtype == "q4k" or qtype == "q5k":
        d, dmin = f16(raw[:, 0:2]), f16(raw[:, 2:4])
        sc, mn = scale_min_k4(raw[:, 4:16])
        qs = raw[:, 48:176] if qtype == "q5k" else raw[:, 16:144]
        qh = raw[:, 16:48] if qtype == "q5k" else None
        for g in range(4):
            q = qs[:, 32 * g:32 * g + 32]
            lo, hi = (q & 0xF).astype(F), (q >> 4).astype(F)
            if qh is not None:
                lo = lo + np.where(qh & (1 << (2 * g)), F(16), F(0))
                hi = hi + np.where(qh & (2 << (2 * g)), F(16), F(0))
            d1, m1 = (d * sc[:, 2 * g]).astype(F), (dmin * mn[:, 2 * g]).astype(F)
            d2, m2 = (d * sc[:, 2 * g + 1]).astype(F), (dmin * mn[:, 2 * g + 1]).astype(F)
            out[:, 64 * g:64 * g + 32] = (d1[:, None] * lo).astype(F) - m1[:, None]
            out[:, 64 * g + 32:64 * g + 64] = (d2[:, None] * hi).astype(F) - m2[:, None]
    elif qtype == "q6k":
        ql, qh, sc, d = raw[:, 0:128], raw[:, 128:192], raw[:, 192:208].view(np.int8).astype(F), f16(raw[:, 208:210])
        for h in range(2):
            l_, h_ = ql[:, 64 * h:64 * h + 64], qh[:, 32 * h:32 * h + 32]
            q = [(l_[:, :32] & 0xF) | ((h_ & 3) << 4), (l_[:, 32:] & 0xF) | (((h_ >> 2) & 3) << 4),
                 (l_[:, :32] >> 4) | (((h_ >> 4) & 3) << 4), (l_[:, 32:] >> 4) | (((h_ >> 6) & 3) << 4)]
            for j in range(4):
                qq = q[j].astype(np.int8).astype(F) - F(32)
                s = np.repeat(sc[:, 8 * h + 2 * j:8 * h + 2 * j + 2], 16, axis=1)
                out[:, 128 * h + 32 * j:128 * h + 32 * j + 32] = ((d[:, None] * s).astype(F) * qq).astype(F)
    elif qtype == "q8k":
        d = raw[:, 0:4].copy().view(np.float32).reshape(-1)
        out = (d[:, None] * raw[:, 4:260].view(np.int8).astype(F)).astype(F)
    elif qtype == "q2k":
        sc, qs, d, dmin = raw[:, 0:16], raw[:, 16:80], f16(raw[:, 80:82]), f16(raw[:, 82:84])
        for h in range(2):
            for j in range(4):
                for half in range(2):
                    s = sc[:, 8 * h + 2 * j + half]
                    dl, ml = (d * (s & 0xF).astype(F)).astype(F), (dmin * (s >> 4).astype(F)).astype(F)
                    q = ((qs[:, 32 * h + 16 * half:32 * h + 16 * half + 16] >> (2 * j)) & 3).astype(F)
                    o = 128 * h + 32 * j + 16 * half
                    out[:, o:o + 16] = (dl[:, None] * q).astype(F) - ml[:, None]
    else:  # q3k
        hm, qs, s12, d = raw[:, 0:32], raw[:, 32:96], raw[:, 96:108], f16(raw[:, 108:110])
        sc = np.zeros((40, 16), np.int32)
        for j in range(16):
            lo = (s12[:, j] & 0xF) if j < 8 else (s12[:, j - 8] >> 4)
            sc[:, j] = (lo | (((s12[:, 8 + j % 4] >> (2 * (j // 4))) & 3) << 4)).astype(np.int32) - 32
        for h in range(2):
            for j in range(4):
                for half in range(2):
                    dl = (d * sc[:, 8 * h + 2 * j + half].astype(F)).astype(F)
                    cols = slice(16 * half, 16 * half + 16)
                    q = ((qs[:, 32 * h:32 * h + 32][:, cols] >> (2 * j)) & 3).astype(np.int32)
                    q = q - np.where(hm[:, cols] & (1 << (4 * h + j)), 0, 4)
                    o = 128 * h + 32 * j + 16 * half
                    out[:, o:o + 16] = (dl[:, None] * q.astype(F)).astype(F)
    assert np.array_equal(out.view(np.uint32), got.view(np.uint32))


# ------------------------------------------------------------------------------------------------
# GPU
# ------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("qtype", KQ)
def test_gpu_dequantize_kats_and_random_blocks(cb, kats, qtype):
    gq = getattr(cb.GgmlDType, qtype.upper())
    k = kats[f"quantize_{qtype}"]
    src = ramp_vector(k["bound"], k["size"])
    blocks = oracle.quantize(src, qtype)  # the CPU writer of the format
    q = cb.QTensor.from_raw(torch.from_numpy(blocks), gq, (k["size"],), device="cuda")
    got = q.dequantize()
    want = np.asarray([float(v) for v in k["dequantized_points_rounded_3"]], np.float32)
    assert np.array_equal(round3(got.cpu().numpy()[k["points"]]), want)
    assert np.array_equal(bits(got), oracle.dequantize(blocks, qtype).view(np.uint32))
    assert np.array_equal(bits(q.dequantize_f16()), bits(got.to(torch.float16)))  # diff == 0 in candle's tests
    rng = np.random.default_rng(17)
    raw = make_kq_blocks(rng, qtype, 333).reshape(-1)
    q = cb.QTensor.from_raw(torch.from_numpy(raw), gq, (333 * 256,), device="cuda")
    f32 = oracle.dequantize(raw, qtype)
    for dt, tdt in (("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)):
        assert np.array_equal(to_oracle(q.dequantize(tdt)), oracle.cast_from_f32(f32, dt)), dt


@pytest.mark.gpu
@pytest.mark.parametrize("qtype", KQ)
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_gpu_lookup_and_lookup_norm(cb, qtype, dtype):
    gq = getattr(cb.GgmlDType, qtype.upper())
    rng = np.random.default_rng(23)
    vocab, hidden = 200, 1024
    table = make_kq_blocks(rng, qtype, vocab * hidden // 256).reshape(vocab, -1)
    ids = rng.integers(0, vocab, size=(3, 50)).astype(np.uint32)
    q = cb.QTensor.from_raw(torch.from_numpy(table), gq, (vocab, hidden), device="cuda")
    tdt = torch.float32 if dtype == "f32" else torch.bfloat16
    rows = oracle.qembedding(table, qtype, ids, dtype)
    assert np.array_equal(to_oracle(q.embedding(ids_tensor(ids), tdt)), rows)
    # a vocabulary shard: ids outside it give rows of zero bits
    part = q_part = cb.QTensor.from_raw(torch.from_numpy(table[50:150]), gq, (100, hidden), device="cuda")
    got = to_oracle(part.embedding(ids_tensor(ids), tdt, vocab_range=(50, 150), vocab=vocab))
    owned = (ids >= 50) & (ids < 150)
    assert np.array_equal(got[owned], rows[owned])
    assert not got[~owned].view(np.uint8).any()
    del q_part
    alpha = randn(rng, (hidden,), dtype, 1.0, 0.1)
    y, g = cb.qembedding_rms_norm(q, ids_tensor(ids), from_oracle(alpha, dtype), 1e-5, return_gathered=True)
    assert np.array_equal(to_oracle(g), rows)
    assert np.array_equal(to_oracle(y), oracle.rms_norm(rows, alpha, 1e-5, dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("qtype", KQ)
def test_gpu_lookup_norm_long_rows(cb, qtype, dtype):
    # Lookup + RMS norm at the row lengths of real tables, with the gathered rows returned too; special
    # rows: a super-block of zero bytes (exact zeros) and a row made of one repeated super-block.
    gq = getattr(cb.GgmlDType, qtype.upper())
    rng = np.random.default_rng(31)
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float16
    for vocab, hidden, n in [(64, 2048, 300), (40, 4096, 257), (24, 8192, 130)]:
        table = make_kq_blocks(rng, qtype, vocab * hidden // 256).reshape(vocab, -1)
        bb = oracle.BLOCK_BYTES[qtype]
        table[1, :bb] = 0                      # a super-block of zeros
        table[2] = np.tile(table[2, :bb], hidden // 256)
        ids = rng.integers(0, vocab, size=(n,)).astype(np.uint32)
        ids[:3] = [1, 2, 1]
        alpha = randn(rng, (hidden,), dtype, 1.0, 0.1)
        rows = oracle.qembedding(table, qtype, ids, dtype)
        want = oracle.rms_norm(rows, alpha, 1e-5, dtype)
        q = cb.QTensor.from_raw(torch.from_numpy(table), gq, (vocab, hidden), device="cuda")
        y, g = cb.qembedding_rms_norm(q, ids_tensor(ids), from_oracle(alpha, dtype), 1e-5, return_gathered=True)
        assert y.dtype == tdt
        assert np.array_equal(to_oracle(g), rows)
        assert np.array_equal(to_oracle(y), want), (qtype, dtype, hidden)
        # the norm forced onto its lane-per-row kernel: the same bits
        y2 = cb.qembedding_rms_norm(q, ids_tensor(ids), from_oracle(alpha, dtype), 1e-5, flags=cb.ops.FLAG_FORCE_LANEROW)
        assert torch.equal(y2.view(torch.int16), y.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("qtype", ["q4k", "q6k"])
def test_gpu_single_launch_lookup_norm_on_a_vocab_shard(cb, qtype):
    # A slice of the vocabulary: ids outside it are rows of zeros going into the norm, an id outside the
    # whole vocabulary is reported and its row left alone.  The single-launch kernel and the forced
    # two-launch route (lookup, then the dense norm) must agree bit for bit on every other row.
    gq = getattr(cb.GgmlDType, qtype.upper())
    rng = np.random.default_rng(41)
    vocab, hidden, n = 96, 2048, 500
    table = make_kq_blocks(rng, qtype, vocab * hidden // 256).reshape(vocab, -1)
    ids = rng.integers(0, vocab, size=(n,)).astype(np.int64)
    ids[7] = vocab + 5
    alpha = from_oracle(randn(rng, (hidden,), "bf16", 1.0, 0.1), "bf16")
    part = cb.QTensor.from_raw(torch.from_numpy(table[32:64]), gq, (32, hidden), device="cuda")
    kw = dict(vocab_range=(32, 64), vocab=vocab, check=False)
    st1, st2 = cb.ops.new_status("cuda"), cb.ops.new_status("cuda")
    y1 = cb.qembedding_rms_norm(part, ids_tensor(ids), alpha, 1e-5, status=st1, **kw)
    y2 = cb.qembedding_rms_norm(part, ids_tensor(ids), alpha, 1e-5, status=st2, flags=cb.ops.FLAG_FORCE_LANEROW, **kw)
    torch.cuda.synchronize()
    keep = np.ones(n, bool)
    keep[7] = False
    keep_t = torch.from_numpy(keep).cuda()
    assert torch.equal(y1[keep_t].view(torch.int16), y2[keep_t].view(torch.int16))
    for st in (st1, st2):
        assert int(st[0].item()) & 0xFFFFFFFF == 1  # CB200_STATUS_INVALID_INDEX
    owned = (ids >= 32) & (ids < 64) & keep
    rows = oracle.qembedding(table, qtype, ids[owned], "bf16")
    assert np.array_equal(to_oracle(y1[torch.from_numpy(owned).cuda()]), oracle.rms_norm(rows, to_oracle(alpha), 1e-5, "bf16"))
