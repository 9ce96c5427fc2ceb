"""The norm's neighbours in a transformer block: ``softmax_last_dim`` (candle-nn/src/ops.rs:289-435),
``rope_i`` / ``rope`` / ``rope_thd`` (candle-nn/src/rotary_emb.rs) and the norm of selected rows only
(the final-norm -> last-token slice of candle-transformers/src/models/quantized_llama.rs:507-508).

CPU part: the oracle against candle's own known answers (candle-nn/tests/ops.rs:9-48, 150-156) and
against the composite "slow" rope formulas candle's tests compare the fused ops with (:158-240).
GPU part: the kernels against the oracle.  rope and the norm of selected rows are bit-exact; softmax
is held to the stated tolerances (1e-5 f32, 1e-2 f16 / bf16) and, beyond that, to agreement in all
but a handful of elements, because exp comes from two different math libraries (the host's expf in
the oracle as in candle, a correctly rounded exp on the device)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import round4
from helpers import TORCH_DT, bits, from_oracle, ids_tensor, randn, stable_seed, to_oracle

TOL = {"f32": 1e-5, "f16": 1e-2, "bf16": 1e-2}


def f32(a):
    return np.asarray(a, dtype=np.float32)


def test_softmax_kats_on_the_oracle(kats):
    k = kats["softmax"]
    x = np.log(f32(k["data"]))
    assert np.array_equal(round4(oracle.softmax_last_dim(x, "f32")), f32(k["expected_last_dim_round4"]))
    # the other two dims of the same test, through a transpose: softmax(x, dim) = softmax_last_dim on dim moved last
    for dim, key in ((0, "expected_dim0_round4"), (1, "expected_dim1_round4")):
        y = np.moveaxis(oracle.softmax_last_dim(np.ascontiguousarray(np.moveaxis(x, dim, -1)), "f32"), -1, dim)
        assert np.array_equal(round4(y), f32(k[key]))
    k = kats["softmax_numerical_stability"]
    assert np.array_equal(oracle.softmax_last_dim(f32(k["x"]), "f32"), f32(k["expected"]))


def rope_slow_numpy(x, cos, sin, interleaved):
    """rope_slow / rope_i_slow of candle-nn/src/rotary_emb.rs:231-251, 492-503 in f32."""
    t = x.shape[2]
    cos, sin = cos[:t], sin[:t]
    if interleaved:
        x0, x1 = x[..., 0::2], x[..., 1::2]
        y0 = (x0 * cos).astype(np.float32) - (x1 * sin).astype(np.float32)
        y1 = (x0 * sin).astype(np.float32) + (x1 * cos).astype(np.float32)
        return np.stack([y0, y1], axis=-1).reshape(x.shape).astype(np.float32)
    c, s = np.concatenate([cos, cos], -1), np.concatenate([sin, sin], -1)
    d = x.shape[-1]
    rot = np.concatenate([-x[..., d // 2:], x[..., :d // 2]], -1)
    return ((x * c).astype(np.float32) + (rot * s).astype(np.float32)).astype(np.float32)


@pytest.mark.parametrize("name", ["ropei", "rope", "rope_thd"])
def test_rope_fused_equals_slow_on_the_oracle(kats, name):
    # candle-nn/tests/ops.rs:158-240: sum |fused - slow| == 0 on the CPU.  The `rand` crate's stream
    # cannot be reproduced; a numpy generator with the same seed value and distribution stands in.
    b, h, t, d = kats[name]["b_size_num_head_seq_len_head_dim"]
    rng = np.random.default_rng(299792458)
    x = rng.random((b, h, t, d), dtype=np.float32)
    cos, sin = rng.random((t, d // 2), dtype=np.float32), rng.random((t, d // 2), dtype=np.float32)
    if name == "ropei":
        got, want = oracle.rope("rope_i", x, cos, sin, "f32"), rope_slow_numpy(x, cos, sin, True)
    elif name == "rope":
        got, want = oracle.rope("rope", x, cos, sin, "f32"), rope_slow_numpy(x, cos, sin, False)
    else:
        xt = np.ascontiguousarray(x.transpose(0, 2, 1, 3))
        got = oracle.rope("rope_thd", xt, cos, sin, "f32").transpose(0, 2, 1, 3)
        want = rope_slow_numpy(x, cos, sin, False)
    assert np.abs(got - want).sum() == kats[name]["fused_vs_slow_sum_abs_diff"]


# ------------------------------------------------------------------------------------------------
# GPU
# ------------------------------------------------------------------------------------------------
@pytest.mark.gpu
def test_gpu_softmax_kats(cb, kats):
    k = kats["softmax"]
    x = torch.log(torch.tensor(k["data"], dtype=torch.float32, device="cuda"))
    y = cb.softmax_last_dim(x)
    assert np.array_equal(round4(y.cpu().numpy()), f32(k["expected_last_dim_round4"]))
    k = kats["softmax_numerical_stability"]
    y = cb.softmax_last_dim(torch.tensor(k["x"], dtype=torch.float32, device="cuda"))
    assert np.array_equal(y.cpu().numpy(), f32(k["expected"]))


SOFTMAX_SHAPES = [(1, 1), (3, 7), (5, 31), (4, 33), (9, 100), (64, 128), (40, 1000), (2, 8, 64, 64), (33, 4096), (3, 40000)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", SOFTMAX_SHAPES)
def test_gpu_softmax_matches_oracle(cb, dtype, shape):
    rng = np.random.default_rng(stable_seed(dtype, shape))
    x = randn(rng, shape, dtype, 0.0, 3.0)
    if len(shape) == 4:  # attention scores with a causal mask: -inf above the diagonal
        xf = oracle.cast_to_f32(x, dtype)
        xf[..., np.triu_indices(shape[-1], 1)[0], np.triu_indices(shape[-1], 1)[1]] = -np.inf
        x = xf if dtype == "f32" else oracle.cast_from_f32(xf, dtype)
    want = oracle.softmax_last_dim(x, dtype)
    got = cb.softmax_last_dim(from_oracle(x, dtype))
    g, w = oracle.cast_to_f32(to_oracle(got), dtype), oracle.cast_to_f32(want, dtype)
    assert np.abs(g - w).max() <= TOL[dtype]
    same = bits(got) == (want.view(np.uint32) if dtype == "f32" else want)
    # exp comes from two math libraries: allow the rare last-bit disagreement, nothing systematic
    if dtype == "f32":
        assert np.abs(g - w).max() <= 2.0 ** -22
        assert (~same).sum() <= max(2, 0.03 * same.size), f"{(~same).sum()} of {same.size} elements differ"
    else:
        assert same.mean() > 0.999, f"{(~same).sum()} of {same.size} elements differ"


@pytest.mark.gpu
def test_gpu_softmax_f32_staged_and_scalar_kernels_agree(cb):
    # Two kernels, two ways to the once-rounded exp (a table-driven double-precision evaluation with a
    # rounding check against the library's exp): bit-equal on rows whose x - max spans the whole range
    # down to results that underflow.  A tensor 4 bytes off 16-byte alignment takes the scalar kernel.
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    rows, n = 2048, 4096
    scale = torch.logspace(-3, 2, rows, device="cuda").unsqueeze(1)  # row spreads from 1e-3 to 100
    x = torch.randn(rows, n, device="cuda", generator=g) * scale
    x[::7, 5] = float("-inf")
    x[3::11, 9] = float("nan")
    store = torch.empty(rows * n + 1, device="cuda")
    xu = store[1:].view(rows, n)
    xu.copy_(x)
    assert x.data_ptr() % 16 == 0 and xu.data_ptr() % 16 == 4
    ya, yu = cb.softmax_last_dim(x), cb.softmax_last_dim(xu)
    a, u = ya.view(torch.int32), yu.view(torch.int32)
    nan = torch.isnan(ya)
    assert torch.equal(nan, torch.isnan(yu))
    assert torch.equal(a[~nan], u[~nan])
    # and both are the correctly rounded exp: numpy's double-precision exp rounded to f32
    xs = x[100].cpu().numpy()
    e = np.exp((xs - xs.max()).astype(np.float32).astype(np.float64)).astype(np.float32)  # (x - max) is an f32 value
    tot = np.float32(oracle.avx_vec_sum(e))
    assert np.array_equal((e / tot).astype(np.float32).view(np.uint32), ya[100].cpu().numpy().view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("n", [2048, 136])
def test_gpu_softmax16_staged_and_scalar_kernels_agree(cb, dtype, n):
    # The staged kernel takes T(exp(T(x - max))) from a table over the magnitudes that matter and divides
    # by reciprocal (bf16) or in three instructions (f16); the scalar kernel evaluates every element and
    # divides for real.  Bit-equal on rows that reach every corner: spreads from 1e-3 to beyond the
    # underflow point (the table's two ends, results that are subnormal in T, rows whose quotients could
    # be), -inf entries, NaN entries, rows of one repeated value, rows that are all -inf.
    tdt = TORCH_DT[dtype]
    g = torch.Generator(device="cuda")
    g.manual_seed(11 + n)
    rows = 1536
    scale = torch.logspace(-3, 2.1, rows, device="cuda").unsqueeze(1)
    x = (torch.randn(rows, n, device="cuda", generator=g) * scale).to(tdt)
    x[::7, 5] = float("-inf")
    x[3::11, 9] = float("nan")
    x[4::97] = 1.5
    x[5::101] = float("-inf")
    x[6::103, : n // 2] = -30000.0 if dtype == "f16" else -1e30
    store = torch.empty(rows * n + 8, dtype=tdt, device="cuda")
    xu = store[1:1 + rows * n].view(rows, n)
    xu.copy_(x)
    assert x.data_ptr() % 16 == 0 and xu.data_ptr() % 16 == 2
    ya, yu = cb.softmax_last_dim(x), cb.softmax_last_dim(xu)
    nan = torch.isnan(ya)
    assert torch.equal(nan, torch.isnan(yu))
    a, u = ya.view(torch.int16), yu.view(torch.int16)
    assert torch.equal(a[~nan], u[~nan]), f"{(a[~nan] != u[~nan]).sum().item()} elements differ"
    # and a slice of ordinary rows against the oracle, within the stated tolerance
    want = oracle.cast_to_f32(oracle.softmax_last_dim(to_oracle(x[600:700]), dtype), dtype)
    got = oracle.cast_to_f32(to_oracle(ya[600:700]), dtype)
    ok = ~np.isnan(want)
    assert np.abs(got[ok] - want[ok]).max() <= TOL[dtype]


ROPE_SHAPES = [(2, 5, 10, 16), (1, 3, 7, 6), (2, 8, 33, 128), (1, 32, 64, 64), (3, 2, 5, 2)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", ROPE_SHAPES)
@pytest.mark.parametrize("variant", ["rope_i", "rope", "rope_thd"])
def test_gpu_rope_matches_oracle(cb, variant, shape, dtype):
    rng = np.random.default_rng(stable_seed(variant, shape, dtype))
    b, h, t, d = shape
    xs = (b, t, h, d) if variant == "rope_thd" else shape
    x = randn(rng, xs, dtype)
    extra = 3  # cos / sin may hold more positions than the sequence uses
    cos, sin = randn(rng, (t + extra, d // 2), dtype), randn(rng, (t + extra, d // 2), dtype)
    want = oracle.rope(variant, x, cos, sin, dtype)
    got = getattr(cb, variant)(from_oracle(x, dtype), from_oracle(cos, dtype), from_oracle(sin, dtype))
    assert np.array_equal(bits(got), want.view(np.uint32) if dtype == "f32" else want)


@pytest.mark.gpu
def test_gpu_rope_kats_and_errors(cb, kats):
    b, h, t, d = kats["rope"]["b_size_num_head_seq_len_head_dim"]
    rng = np.random.default_rng(299792458)
    x = rng.random((b, h, t, d), dtype=np.float32)
    cos, sin = rng.random((t, d // 2), dtype=np.float32), rng.random((t, d // 2), dtype=np.float32)
    xt, ct, st = (torch.from_numpy(a).cuda() for a in (x, cos, sin))
    assert np.abs(cb.rope(xt, ct, st).cpu().numpy() - rope_slow_numpy(x, cos, sin, False)).sum() == 0.0
    assert np.abs(cb.rope_i(xt, ct, st).cpu().numpy() - rope_slow_numpy(x, cos, sin, True)).sum() == 0.0
    thd = cb.rope_thd(xt.transpose(1, 2).contiguous(), ct, st).transpose(1, 2)
    assert np.abs(thd.cpu().numpy() - rope_slow_numpy(x, cos, sin, False)).sum() == 0.0
    with pytest.raises(cb.CandleError, match="inconsistent last dim size in rope"):
        cb.rope(xt, ct[:, :4], st)
    with pytest.raises(cb.CandleError, match="inconsistent last dim size in rope"):
        cb.rope(xt, ct[: t - 1], st[: t - 1])
    with pytest.raises(cb.CandleError, match="xs has to be contiguous in rope"):
        cb.rope(xt.transpose(1, 2), ct, st)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_gpu_norm_of_selected_rows(cb, dtype):
    """Final norm -> last token: only the selected rows are normalised, values as the full norm's."""
    rng = np.random.default_rng(77)
    b, t, hidden = 6, 50, 4096
    x, a = randn(rng, (b * t, hidden), dtype), randn(rng, (hidden,), dtype, 1.0, 0.1)
    last = (np.arange(b) * t + t - 1).astype(np.uint32)
    full = oracle.rms_norm(x, a, 1e-5, dtype)
    got = cb.rms_norm_rows(from_oracle(x, dtype), ids_tensor(last), from_oracle(a, dtype), 1e-5)
    assert tuple(got.shape) == (b, hidden)
    assert np.array_equal(to_oracle(got), full[last])
    with pytest.raises(cb.InvalidIndex):
        cb.rms_norm_rows(from_oracle(x, dtype), ids_tensor(np.asarray([b * t], np.uint32)), from_oracle(a, dtype), 1e-5)
