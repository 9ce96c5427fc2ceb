"""candle's composite ("slow") norm path: ``LayerNorm::forward`` off the fused path
(candle-nn/src/layer_norm.rs:108-136) and ``ops::rms_norm_slow`` / ``layer_norm_slow``
(candle-nn/src/ops.rs:628-639, 876-894).

CPU part: the C restatement against candle's own golden values for the slow formulas
(candle-nn/tests/ops.rs:55-78, 101-125) and against an independent numpy statement of the AVX
summation order.  GPU part: the kernel against the restatement, bit for bit (the kernel follows the
same AVX order), plus the stated tolerances, plus the module dispatch."""
import numpy as np
import pytest
import torch

import oracle
from conftest import round4
from helpers import bits, from_oracle, randn, stable_seed, to_oracle

TOL = {"f32": 1e-5, "f16": 1e-2, "bf16": 1e-2}


def f32(a):
    return np.asarray(a, dtype=np.float32)


def numpy_avx_sum(row):
    """vec_sum of candle-core/src/cpu/mod.rs:113-135 with the AVX fold of cpu/avx.rs:54-66."""
    row = np.asarray(row, np.float32)
    k = row.size
    np_ = k & ~31
    acc = np.zeros(32, np.float32)
    for i in range(0, np_, 32):
        acc = (acc + row[i:i + 32]).astype(np.float32)
    a = acc.reshape(4, 8)
    r8 = ((a[0] + a[1]).astype(np.float32) + (a[2] + a[3]).astype(np.float32)).astype(np.float32)
    t0 = (r8[:4] + r8[4:]).astype(np.float32)
    b = np.float32(np.float32(t0[0] + t0[1]) + np.float32(t0[2] + t0[3]))
    for i in range(np_, k):
        b = np.float32(b + row[i])
    return b


@pytest.mark.parametrize("n", [1, 3, 31, 32, 33, 64, 100, 768, 1000, 4096])
def test_avx_vec_sum_order(n):
    rng = np.random.default_rng(n)
    row = rng.standard_normal(n).astype(np.float32)
    assert np.float32(oracle.avx_vec_sum(row)) == numpy_avx_sum(row)


def test_slow_kats_through_the_c_restatement(kats):
    k = kats["rms_norm"]
    y = oracle.norm_slow(f32(k["x"]), f32(k["alpha"]), None, k["eps"], "f32", remove_mean=False)
    assert np.array_equal(round4(y), f32(k["expected_slow_round4"]))
    fused = oracle.rms_norm(f32(k["x"]), f32(k["alpha"]), k["eps"], "f32")
    assert np.abs(fused - y).sum() < 1e-5  # candle-nn/tests/ops.rs:73-76
    k = kats["layer_norm"]
    y = oracle.norm_slow(f32(k["x"]), f32(k["alpha"]), f32(k["beta"]), k["eps"], "f32", remove_mean=True)
    assert np.array_equal(round4(y), f32(k["expected_slow_round4"]))
    fused = oracle.layer_norm(f32(k["x"]), f32(k["alpha"]), f32(k["beta"]), k["eps"], "f32")
    assert np.abs(fused - y).sum() < 1e-5


@pytest.mark.parametrize("name", ["rms_norml", "layer_norml"])
def test_norml_fused_vs_slow_restated(kats, name):
    # candle-nn/tests/ops.rs:80-99, 127-147 with both sides from the C restatement
    k = kats[name]
    x = np.random.default_rng(299792458).random(k["shape"], dtype=np.float32)
    n = x.shape[-1]
    ones, zeros = np.ones(n, np.float32), np.zeros(n, np.float32)
    if name == "rms_norml":
        fused, slow = oracle.rms_norm(x, ones, k["eps"], "f32"), oracle.norm_slow(x, ones, None, k["eps"], "f32", False)
    else:
        fused, slow = oracle.layer_norm(x, ones, zeros, k["eps"], "f32"), oracle.norm_slow(x, ones, zeros, k["eps"], "f32", True)
    assert np.abs(fused - slow).max() < k["max_abs_fused_vs_slow"]


def test_slow_chain_against_numpy_statement():
    rng = np.random.default_rng(5)
    for dtype in ("f32", "bf16", "f16"):
        x, w, b = randn(rng, (6, 100), dtype), randn(rng, (100,), dtype, 1.0, 0.1), randn(rng, (100,), dtype, 0.0, 0.1)
        got = oracle.norm_slow(x, w, b, 1e-5, dtype, True)
        xf = oracle.cast_to_f32(x, dtype)
        inv_n = np.float32(1.0 / 100)
        out = np.empty_like(xf)
        for r in range(6):
            mean = np.float32(np.float32(numpy_avx_sum(xf[r]) * inv_n) + np.float32(0))
            xc = (xf[r] - mean).astype(np.float32)
            q = numpy_avx_sum((xc * xc).astype(np.float32))
            d = np.sqrt(np.float32(np.float32(np.float32(q * inv_n) + np.float32(0)) * np.float32(1) + np.float32(1e-5)))
            out[r] = (xc / d).astype(np.float32)
        t = oracle.cast_from_f32(out, dtype) if dtype != "f32" else out
        wf, bf = oracle.cast_to_f32(w, dtype), oracle.cast_to_f32(b, dtype)
        t = oracle.cast_from_f32((oracle.cast_to_f32(t, dtype) * wf).astype(np.float32), dtype)
        t = oracle.cast_from_f32((oracle.cast_to_f32(t, dtype) + bf).astype(np.float32), dtype)
        assert np.array_equal(np.asarray(t).view(np.uint8), np.asarray(got).view(np.uint8)), dtype


# ------------------------------------------------------------------------------------------------
# GPU
# ------------------------------------------------------------------------------------------------
def check(got: torch.Tensor, want: np.ndarray, dtype: str):
    g = to_oracle(got)
    assert np.abs(oracle.cast_to_f32(g, dtype) - oracle.cast_to_f32(want, dtype)).max() <= TOL[dtype]
    same = bits(got) == (want.view(np.uint32) if dtype == "f32" else want)
    assert same.all(), f"{(~same).sum()} of {same.size} elements differ in bits"


SLOW_SHAPES = [(1, 8), (7, 3), (5, 31), (3, 33), (9, 200), (33, 768), (12, 4096), (2, 3, 8192), (3, 1000)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", SLOW_SHAPES)
@pytest.mark.parametrize("form", ["rms", "ln", "ln_no_bias"])
def test_slow_norm_matches_oracle(cb, dtype, shape, form):
    rng = np.random.default_rng(stable_seed(dtype, shape, form))
    n = shape[-1]
    x, w, b = randn(rng, shape, dtype), randn(rng, (n,), dtype, 1.0, 0.1), randn(rng, (n,), dtype, 0.0, 0.1)
    eps = 1e-5
    xt, wt, bt = from_oracle(x, dtype), from_oracle(w, dtype), from_oracle(b, dtype)
    if form == "rms":
        want = oracle.norm_slow(x, w, None, eps, dtype, False)
        check(cb.rms_norm_slow(xt, wt, eps), want, dtype)
        check(cb.LayerNorm.rms_norm(wt, eps).forward(xt), want, dtype)
        check(cb.RmsNorm(wt, eps).forward_diff(xt), want, dtype)
    elif form == "ln":
        want = oracle.norm_slow(x, w, b, eps, dtype, True)
        check(cb.layer_norm_slow(xt, wt, bt, eps), want, dtype)
    else:
        want = oracle.norm_slow(x, w, None, eps, dtype, True)
        check(cb.LayerNorm.new_no_bias(wt, eps).forward(xt), want, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_module_dispatch_follows_candle(cb, dtype):
    """Contiguous + remove_mean + bias -> fused op; a transposed (non-contiguous) input -> the
    composite chain on a contiguous copy; RmsNorm::forward is the only user of the fused rms op."""
    rng = np.random.default_rng(11)
    x = randn(rng, (64, 512), dtype)
    w, b = randn(rng, (512,), dtype, 1.0, 0.1), randn(rng, (512,), dtype, 0.0, 0.1)
    xt, wt, bt = from_oracle(x, dtype), from_oracle(w, dtype), from_oracle(b, dtype)
    ln = cb.LayerNorm.new(wt, bt, 1e-5)
    check(ln.forward(xt), oracle.layer_norm(x, w, b, 1e-5, dtype), dtype)
    # non-contiguous view of the same values: [512, 64] storage read as its transpose
    xs = xt.t().contiguous().t()
    assert not xs.is_contiguous() and torch.equal(xs, xt)
    check(ln.forward(xs), oracle.norm_slow(x, w, b, 1e-5, dtype, True), dtype)
    rn = cb.RmsNorm(wt, 1e-5)
    check(rn.forward(xt), oracle.rms_norm(x, w, 1e-5, dtype), dtype)
    check(rn.forward(xs), oracle.norm_slow(x, w, None, 1e-5, dtype, False), dtype)
    check(rn.into_inner().forward(xt), oracle.norm_slow(x, w, None, 1e-5, dtype, False), dtype)


@pytest.mark.gpu
def test_fused_and_slow_rms_differ_in_bf16_where_candles_do(cb):
    rng = np.random.default_rng(3)
    x, w = randn(rng, (256, 4096), "bf16"), randn(rng, (4096,), "bf16", 1.0, 0.1)
    xt, wt = from_oracle(x, "bf16"), from_oracle(w, "bf16")
    fused, slow = cb.RmsNorm(wt, 1e-5).forward(xt), cb.LayerNorm.rms_norm(wt, 1e-5).forward(xt)
    want_fused, want_slow = oracle.rms_norm(x, w, 1e-5, "bf16"), oracle.norm_slow(x, w, None, 1e-5, "bf16", False)
    differ = to_oracle(fused) != to_oracle(slow)
    assert differ.any(), "three roundings and one rounding cannot agree everywhere at this size"
    assert np.array_equal(differ, want_fused != want_slow)
