"""The benchmark's configurations at their full sizes, every row against the CPU oracle, through the
front ends over the C ABI: C1 (f32 table 32000 x 4096, 4096 ids, lookup + RMS norm), C2 (layer norm +
residual bf16, 16384 x 768), C3 (Q8_0 table 128256 x 4096, 65536 Zipf ids, lookup + RMS norm, ids in
rank order and permuted over the table) and the C5 row ladder at 8192 columns (1 ... 8192 rows; the
65536-row case is covered through a size-independent property: its rows are the 4096-row block
repeated, so every block of the result must equal the first, which is compared with the oracle).
Inputs are seeded synthetic data with the configurations' shapes and value distributions."""
import numpy as np
import pytest
import torch

import oracle
from helpers import from_oracle, ids_tensor, make_qtable, randn, to_oracle

pytestmark = pytest.mark.gpu
THREADS = 0  # the oracle's default: all cores


def zipf_ids(rng, vocab, n, s=1.1):
    p = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** s
    p /= p.sum()
    return rng.choice(vocab, size=n, p=p).astype(np.uint32)


def test_c1_f32_table_lookup_rms_norm_all_rows(cb):
    rng = np.random.default_rng(101)
    vocab, hidden, n = 32000, 4096, 8 * 512
    table = randn(rng, (vocab, hidden), "f32", 0.0, 0.02)
    alpha = randn(rng, (hidden,), "f32", 1.0, 0.1)
    ids = rng.integers(0, vocab, size=(8, 512)).astype(np.uint32)
    want = oracle.rms_norm(oracle.embedding(table, ids), alpha, 1e-5, "f32")
    y = cb.embedding_rms_norm(from_oracle(table, "f32"), ids_tensor(ids), from_oracle(alpha, "f32"), 1e-5)
    assert tuple(y.shape) == (8, 512, hidden)
    assert np.array_equal(to_oracle(y).view(np.uint32), want.view(np.uint32))
    # the two-step form candle runs (Embedding::forward, then rms_norm) gives the same bits
    e = cb.Embedding(from_oracle(table, "f32"), hidden).forward(ids_tensor(ids))
    y2 = cb.rms_norm(e, from_oracle(alpha, "f32"), 1e-5)
    assert torch.equal(y2.view(torch.int32), y.view(torch.int32))


def test_c2_layer_norm_residual_bf16_all_rows(cb):
    rng = np.random.default_rng(102)
    rows, hidden = 16384, 768
    x, res = randn(rng, (rows, hidden), "bf16"), randn(rng, (rows, hidden), "bf16")
    gamma, beta = randn(rng, (hidden,), "bf16", 1.0, 0.1), randn(rng, (hidden,), "bf16", 0.0, 0.1)
    h = oracle.add(x, res, "bf16")
    want = oracle.layer_norm(h, gamma, beta, 1e-12, "bf16")
    y, s = cb.layer_norm(from_oracle(x, "bf16"), from_oracle(gamma, "bf16"), from_oracle(beta, "bf16"), 1e-12,
                         residual=from_oracle(res, "bf16"), return_sum=True)
    assert np.array_equal(to_oracle(s), h)
    assert np.array_equal(to_oracle(y), want)


@pytest.mark.parametrize("permuted", [False, True])
def test_c3_q8_0_table_zipf_lookup_rms_norm_all_rows(cb, permuted):
    rng = np.random.default_rng(103)
    vocab, hidden, n = 128256, 4096, 32 * 2048
    qt = make_qtable(rng, "q8_0", vocab, hidden)
    alpha = randn(rng, (hidden,), "bf16", 1.0, 0.1)
    ids = zipf_ids(rng, vocab, n)
    if permuted:
        ids = rng.permutation(vocab).astype(np.uint32)[ids]
    want = oracle.rms_norm(oracle.qembedding(qt, "q8_0", ids, "bf16"), alpha, 1e-5, "bf16")
    q = cb.QTensor.from_raw(torch.from_numpy(qt), cb.GgmlDType.Q8_0, (vocab, hidden), device="cuda")
    y = cb.qembedding_rms_norm(q, ids_tensor(ids.reshape(32, 2048)), from_oracle(alpha, "bf16"), 1e-5)
    assert tuple(y.shape) == (32, 2048, hidden)
    assert np.array_equal(to_oracle(y).reshape(n, hidden), want)


@pytest.mark.parametrize("rows", [1, 8, 64, 512, 8192])
def test_c5_rms_norm_residual_bf16_row_ladder_all_rows(cb, rows):
    rng = np.random.default_rng(105)
    hidden = 8192
    x, res = randn(rng, (rows, hidden), "bf16"), randn(rng, (rows, hidden), "bf16")
    alpha = randn(rng, (hidden,), "bf16", 1.0, 0.1)
    h = oracle.add(x, res, "bf16")
    want = oracle.rms_norm(h, alpha, 1e-5, "bf16")
    y, s = cb.rms_norm(from_oracle(x, "bf16"), from_oracle(alpha, "bf16"), 1e-5, residual=from_oracle(res, "bf16"),
                       return_sum=True)
    assert np.array_equal(to_oracle(s), h)
    assert np.array_equal(to_oracle(y), want)


def test_c5_full_size_is_the_seeded_block_repeated(cb):
    # 65536 x 8192 with residual: 3.2 GB through the kernel; the inputs are a 4096-row block tiled
    # 16 times, so each block of the output must equal the first, and the first equals the oracle.
    rng = np.random.default_rng(106)
    base, reps, hidden = 4096, 16, 8192
    x, res = randn(rng, (base, hidden), "bf16"), randn(rng, (base, hidden), "bf16")
    alpha = randn(rng, (hidden,), "bf16", 1.0, 0.1)
    want = oracle.rms_norm(oracle.add(x, res, "bf16"), alpha, 1e-5, "bf16")
    xt, rt = from_oracle(x, "bf16").repeat(reps, 1), from_oracle(res, "bf16").repeat(reps, 1)
    y = cb.rms_norm(xt, from_oracle(alpha, "bf16"), 1e-5, residual=rt)
    first = y[:base]
    assert np.array_equal(to_oracle(first), want)
    for k in range(1, reps):
        assert torch.equal(y[k * base:(k + 1) * base].view(torch.int16), first.view(torch.int16)), f"block {k}"
