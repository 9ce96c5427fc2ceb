"""The CPU oracle against every golden vector candle's own tests hold for this path."""
import numpy as np
import pytest
import torch

import oracle
from conftest import round4


def f32(a):
    return np.asarray(a, dtype=np.float32)


def test_rms_norm_kat(kats):
    k = kats["rms_norm"]  # candle-nn/tests/ops.rs:55-78
    y = oracle.rms_norm(f32(k["x"]), f32(k["alpha"]), k["eps"], "f32")
    assert np.array_equal(round4(y), f32(k["expected_round4"]))
    # fused vs the composite "slow" formula: sum |diff| < 1e-5 (same test)
    x = f32(k["x"])
    slow = x / np.sqrt((x * x).sum(-1, keepdims=True, dtype=np.float32) / np.float32(3) + np.float32(k["eps"]))
    slow = slow.astype(np.float32) * f32(k["alpha"])
    assert np.abs(y - slow).sum() < 1e-5
    assert np.array_equal(round4(slow), f32(k["expected_slow_round4"]))


def test_layer_norm_kat(kats):
    k = kats["layer_norm"]  # candle-nn/tests/ops.rs:101-125
    y = oracle.layer_norm(f32(k["x"]), f32(k["alpha"]), f32(k["beta"]), k["eps"], "f32")
    assert np.array_equal(round4(y), f32(k["expected_round4"]))


@pytest.mark.parametrize("name", ["rms_norml", "layer_norml"])
def test_norml_fused_vs_slow(kats, name):
    # candle-nn/tests/ops.rs:80-99,127-147: (24,70,64) uniform[0,1); max |fused - slow| < 1e-5.
    # The `rand` crate's StdRng stream cannot be reproduced here; a numpy generator with the same
    # seed value and distribution stands in.
    k = kats[name]
    rng = np.random.default_rng(299792458)
    x = rng.random(k["shape"], dtype=np.float32)
    n = np.float32(x.shape[-1])
    ones, zeros = np.ones(x.shape[-1], np.float32), np.zeros(x.shape[-1], np.float32)
    if name == "rms_norml":
        y = oracle.rms_norm(x, ones, k["eps"], "f32")
        slow = x / np.sqrt((x * x).sum(-1, keepdims=True, dtype=np.float32) / n + np.float32(k["eps"]))
    else:
        y = oracle.layer_norm(x, ones, zeros, k["eps"], "f32")
        xc = x - x.sum(-1, keepdims=True, dtype=np.float32) / n
        slow = xc / np.sqrt((xc * xc).sum(-1, keepdims=True, dtype=np.float32) / n + np.float32(k["eps"]))
    assert np.abs(y - slow.astype(np.float32)).max() < k["max_abs_fused_vs_slow"]


def test_layer_norm_module_kat(kats):
    k = kats["layer_norm_module"]  # candle-nn/tests/layer_norm.rs:11-55
    for case in k["cases"]:
        x = f32(case["x"])
        h = x.shape[-1]
        w, b = np.full(h, k["w"][0], np.float32), np.full(h, k["b"][0], np.float32)
        y = oracle.layer_norm(x, w, b, k["eps"], "f32")
        if case.get("exact"):
            assert np.array_equal(y.reshape(-1), f32(case["expected"]).reshape(-1))
        else:
            assert np.array_equal(round4(y), f32(case["expected_round4"]))
            mean = (y.sum(-1, keepdims=True, dtype=np.float32) / np.float32(3)).astype(np.float32)
            assert np.array_equal(round4(mean), f32(case["mean_round4"]))
            std = np.sqrt(((y - mean) ** 2).sum(-1, keepdims=True, dtype=np.float32)) / np.float32(3)
            assert np.array_equal(round4(std), f32(case["std_round4"]))


def test_layer_norm_doctest_kat(kats):
    k = kats["layer_norm_doctest"]  # candle-nn/src/layer_norm.rs:7-28
    y = oracle.layer_norm(f32(k["x"]), f32(k["w"]), f32(k["b"]), k["eps"], "f32")
    assert np.array_equal(round4(y), f32(k["expected_round4"]))


def test_embeddings_kat(kats):
    k = kats["embeddings"]  # candle-core/tests/tensor_tests.rs:817-827
    table = f32(k["table"])
    for idt in (np.uint32, np.int64):
        ids = np.asarray(k["ids"], dtype=idt)
        assert np.array_equal(oracle.embedding(table, ids), f32(k["expected"]))
        assert np.array_equal(oracle.index_select(table, ids, 0), f32(k["expected"]))


def test_index_select_kat(kats):
    k = kats["index_select"]  # candle-core/tests/tensor_tests.rs:841-896
    t = np.arange(12, dtype=np.float32).reshape(k["table_arange"])
    assert np.array_equal(t, f32(k["table"]))
    for idt in (np.uint8, np.uint32, np.int64):
        ids = np.asarray(k["ids"], dtype=idt)
        assert np.array_equal(oracle.index_select(t, ids, 1), f32(k["expected_dim1"]))
        assert np.array_equal(oracle.index_select(t, ids, 0), f32(k["expected_dim0"]))
        rep = np.asarray(k["ids_repeated"], dtype=idt)
        assert np.array_equal(oracle.index_select(t, rep, 0), f32(k["expected_repeated_dim0"]))
        ids2 = np.asarray(k["ids2"], dtype=idt)
        assert np.array_equal(oracle.index_select(f32(k["table2"]), ids2, 1), f32(k["expected2_dim1"]))


def test_index_select_invalid_index_and_strided_ids():
    t = np.arange(12, dtype=np.float32).reshape(4, 3)
    with pytest.raises(oracle.InvalidIndex) as e:  # cpu_backend/mod.rs:539-546
        oracle.index_select(t, np.asarray([0, 4], np.uint32), 0)
    assert (e.value.index, e.value.size, e.value.op) == (4, 4, "index-select")
    with pytest.raises(oracle.InvalidIndex):
        oracle.index_select(t, np.asarray([-1], np.int64), 0)
    strided = np.asarray([3, 9, 1, 9, 0, 9], np.uint32)[::2]  # ids stride honoured, :526,538
    assert np.array_equal(oracle.index_select(t, strided, 0), t[[3, 1, 0]])
    assert oracle.index_select(t, np.zeros(0, np.uint32), 0).shape == (0, 3)


def test_quantize_q4_0_kat(kats):
    k = kats["quantize_q4_0"]  # candle-core/tests/quantized_tests.rs:222-254
    src = np.arange(128, dtype=np.float32)
    blocks = oracle.quantize(src, "q4_0")
    assert blocks.shape == (4 * 18,)
    dst = oracle.dequantize(blocks, "q4_0")
    want = np.asarray([float(v) for v in k["dequantized"]], dtype=np.float32)
    assert np.array_equal(dst.view(np.uint32), want.view(np.uint32))  # bit-exact incl. the two -0.0
    # dequantize(..).to_dtype(F16) == dequantize_f16(..) (same test, diff == 0)
    as_f16 = oracle.qembedding(blocks.reshape(1, -1), "q4_0", np.zeros(1, np.uint32), "f16")
    assert np.array_equal(as_f16.reshape(-1), oracle.cast_from_f32(dst, "f16"))


@pytest.mark.parametrize("qtype,bytes_per_block", [("q4_1", 20), ("q5_0", 22), ("q5_1", 24)])
def test_quantize_q4_1_q5_0_q5_1_kats(kats, qtype, bytes_per_block):
    k = kats[f"quantize_{qtype}"]  # candle-core/tests/quantized_tests.rs:256-351
    src = np.arange(128, dtype=np.float32)
    blocks = oracle.quantize(src, qtype)
    assert blocks.shape == (4 * bytes_per_block,)
    dst = oracle.dequantize(blocks, qtype)
    want = np.asarray([float(v) for v in k["dequantized_rounded_3"]], dtype=np.float32)
    # candle's round_vector: (1000. * x).round() / 1000. in f32, half away from zero
    scaled = dst * np.float32(1000.0)
    rounded = (np.sign(scaled) * np.floor(np.abs(scaled) + np.float32(0.5))).astype(np.float32) / np.float32(1000.0)
    assert np.array_equal(rounded, want)
    if qtype == "q5_0":  # the first element is -0.0 in candle's vector
        assert np.signbit(dst[0]) and dst[0] == 0.0
    as_f16 = oracle.qembedding(blocks.reshape(1, -1), qtype, np.zeros(1, np.uint32), "f16")
    assert np.array_equal(as_f16.reshape(-1), oracle.cast_from_f32(dst, "f16"))  # diff == 0 in candle's test


def test_q8_0_roundtrip_error_bound():
    # No golden Q8_0 dequant vector exists in candle; pin the format through quantise->dequantise:
    # |x - dq(q(x))| <= d/2 per element with d = amax/127 rounded to f16.
    rng = np.random.default_rng(0)
    x = rng.standard_normal((64, 256)).astype(np.float32)
    blocks = oracle.quantize(x, "q8_0")
    assert blocks.shape == (64, 8 * 34)
    y = oracle.dequantize(blocks, "q8_0")
    d = blocks.reshape(64, 8, 34)[:, :, :2].copy().view(np.float16).astype(np.float32)  # [64,8,1]
    err = np.abs(x - y).reshape(64, 8, 32)
    assert (err <= 0.5 * d * 1.01 + 127 * np.abs(d) * 2**-11).all()
    # exact reconstruction of the stored integers: y / d is an integer in [-127, 127]
    q = blocks.reshape(64, 8, 34)[:, :, 2:].copy().view(np.int8).astype(np.float32)
    assert np.array_equal(y.reshape(64, 8, 32), q * d)


def test_half_conversions_match_torch():
    rng = np.random.default_rng(1)
    bits = rng.integers(0, 2**32, size=200_000, dtype=np.uint64).astype(np.uint32)
    special = np.asarray(
        [0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0x7F800001, 0x3F808000, 0x3F818000,
         0x3F807FFF, 0x3F808001, 0x33000000, 0x33800000, 0x38800000, 0x387FC000, 0x477FE000, 0x477FF000,
         0x00000001, 0x007FFFFF, 0x00800000, 0x7F7FFFFF],
        dtype=np.uint32,
    )
    x = np.concatenate([bits, special]).view(np.float32)
    finite = np.isfinite(x) | np.isinf(x)
    t = torch.from_numpy(x.copy())
    for dt, tdt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        ours = oracle.cast_from_f32(x, dt)
        theirs = t.to(tdt).view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(ours[finite], theirs[finite])
        nan = ~finite  # NaNs stay NaNs (payload conventions may differ between libraries)
        back = oracle.cast_to_f32(ours, dt)
        assert np.isnan(back[nan]).all()
        assert np.array_equal(
            back[finite].view(np.uint32), t.to(tdt).to(torch.float32).numpy()[finite].view(np.uint32)
        )
    # every f16 / bf16 bit pattern decodes as torch does
    all16 = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    for dt, tdt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        ours = oracle.cast_to_f32(all16, dt)
        theirs = torch.from_numpy(all16.view(np.int16).copy()).view(tdt).to(torch.float32).numpy()
        ok = ~np.isnan(theirs)
        assert np.array_equal(ours[ok].view(np.uint32), theirs[ok].view(np.uint32))
        assert np.isnan(ours[~ok]).all()


def _rms_chain_numpy(x16, a16, eps, to32, from32):
    """Independent numpy statement of the bf16/f16 rms-norm rounding chain (ops.rs:484-495)."""
    x = to32(x16)
    s = np.zeros(x.shape[0], np.float32)
    for c in range(x.shape[1]):  # strictly sequential f32 sum
        s = (s + (x[:, c] * x[:, c]).astype(np.float32)).astype(np.float32)
    m = np.sqrt((s / np.float32(x.shape[1]) + np.float32(eps)).astype(np.float32)).astype(np.float32)
    m = to32(from32(m))
    q = to32(from32((x / m[:, None]).astype(np.float32)))
    return from32((q * to32(a16)[None, :]).astype(np.float32))


@pytest.mark.parametrize("dt,tdt", [("bf16", torch.bfloat16), ("f16", torch.float16)])
def test_half_norms_follow_the_rounding_chain(dt, tdt):
    rng = np.random.default_rng(2)
    to32 = lambda a: oracle.cast_to_f32(a, dt)
    from32 = lambda a: oracle.cast_from_f32(a, dt)
    x = from32(rng.standard_normal((37, 200)).astype(np.float32))
    a = from32((1 + 0.1 * rng.standard_normal(200)).astype(np.float32))
    b = from32((0.1 * rng.standard_normal(200)).astype(np.float32))
    assert np.array_equal(oracle.rms_norm(x, a, 1e-5, dt), _rms_chain_numpy(x, a, 1e-5, to32, from32))
    # layer norm: f32 throughout, one final rounding (ops.rs:709-726)
    xf, af, bf = to32(x), to32(a), to32(b)
    s = np.zeros(37, np.float32)
    s2 = np.zeros(37, np.float32)
    for c in range(200):
        s = (s + xf[:, c]).astype(np.float32)
        s2 = (s2 + (xf[:, c] * xf[:, c]).astype(np.float32)).astype(np.float32)
    mean = s / np.float32(200)
    var = s2 / np.float32(200) - mean * mean
    inv = np.float32(1) / np.sqrt(var + np.float32(1e-5))
    want = from32(((xf - mean[:, None]) * inv[:, None] * af[None, :] + bf[None, :]).astype(np.float32))
    assert np.array_equal(oracle.layer_norm(x, a, b, 1e-5, dt), want)
    # residual add is rounded to T before the norm sees it (op.rs:330)
    r = from32(rng.standard_normal((37, 200)).astype(np.float32))
    h = oracle.add(x, r, dt)
    th = (torch.from_numpy(x.view(np.int16).copy()).view(tdt) + torch.from_numpy(r.view(np.int16).copy()).view(tdt))
    assert np.array_equal(h, th.view(torch.int16).numpy().view(np.uint16))


def test_threads_do_not_change_results():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((64, 512)).astype(np.float32)
    a = rng.standard_normal(512).astype(np.float32)
    assert np.array_equal(oracle.rms_norm(x, a, 1e-5, "f32", threads=1), oracle.rms_norm(x, a, 1e-5, "f32", threads=4))
    assert np.array_equal(
        oracle.layer_norm(x, a, a, 1e-5, "f32", threads=1), oracle.layer_norm(x, a, a, 1e-5, "f32", threads=4)
    )
