"""The give-up paths of the bounded device-side waits, one test per kernel family that waits for
bulk copies (row-slot lookup + norm, streaming norm, whole-row norm with gathered rows, dense
gather, quantised gather).

Nothing is made to fail: the library's self-test hook (``cb200_selftest_wait_expiry``) makes each
mbarrier expect 16 bytes more than its copies deliver and cuts the poll budget to a few dozen, so
the wait runs out on a healthy device.  The kernel must then record ``CB200_STATUS_WAIT_TIMEOUT``,
let its copies land and return; the next ordinary call on the same stream must be bit-exact."""
import numpy as np
import pytest
import torch

import oracle
from helpers import from_oracle, ids_tensor, make_qtable, randn, to_oracle

pytestmark = pytest.mark.gpu

WAIT_TIMEOUT = 2


def expire_then_recover(cb, run, want):
    """run(status) -> output tensor.  First with every wait forced to run out, then normally."""
    from candle_b200 import _cabi
    from candle_b200.ops import new_status

    st = new_status("cuda")
    _cabi.call("cb200_selftest_wait_expiry", 1)
    try:
        run(st)
        torch.cuda.synchronize()
    finally:
        _cabi.call("cb200_selftest_wait_expiry", 0)
    assert int(st[0].item()) & 0xFFFFFFFF == WAIT_TIMEOUT, "the forced expiry was not recorded"
    st.zero_()
    got = run(st)
    torch.cuda.synchronize()
    assert int(st[0].item()) == 0
    assert np.array_equal(to_oracle(got), want), "the call after a timed-out one is not bit-exact"


def test_rowslot_lookup_norm(cb):
    rng = np.random.default_rng(1)
    vocab, hidden = 512, 4096
    qt = make_qtable(rng, "q8_0", vocab, hidden)
    ids = rng.integers(0, vocab, size=2048).astype(np.uint32)
    alpha = randn(rng, (hidden,), "bf16", 1.0, 0.1)
    q = cb.QTensor.from_raw(torch.from_numpy(qt), cb.GgmlDType.Q8_0, (vocab, hidden), device="cuda")
    it, at = ids_tensor(ids), from_oracle(alpha, "bf16")
    want = oracle.rms_norm(oracle.qembedding(qt, "q8_0", ids, "bf16"), alpha, 1e-5, "bf16")
    expire_then_recover(cb, lambda st: cb.qembedding_rms_norm(q, it, at, 1e-5, check=False, status=st), want)


def test_streaming_norm(cb):
    rng = np.random.default_rng(2)
    x, a = randn(rng, (300, 4096), "f32"), randn(rng, (4096,), "f32", 1.0, 0.1)
    xt, at = from_oracle(x, "f32"), from_oracle(a, "f32")
    want = oracle.rms_norm(x, a, 1e-5, "f32")
    expire_then_recover(cb, lambda st: cb.rms_norm(xt, at, 1e-5, status=st), want)


def test_whole_row_norm_with_gathered_rows(cb):
    rng = np.random.default_rng(3)
    table, a = randn(rng, (1000, 64), "f32"), randn(rng, (64,), "f32", 1.0, 0.1)  # 256-byte rows
    ids = rng.integers(0, 1000, size=700).astype(np.uint32)
    tt, at, it = from_oracle(table, "f32"), from_oracle(a, "f32"), ids_tensor(ids)
    want = oracle.rms_norm(oracle.embedding(table, ids), a, 1e-5, "f32")
    expire_then_recover(cb, lambda st: cb.embedding_rms_norm(tt, it, at, 1e-5, check=False, status=st), want)


def test_dense_gather(cb):
    rng = np.random.default_rng(4)
    table = randn(rng, (777, 1024), "f32")  # 4 KB rows: the bulk-copy gather
    ids = rng.integers(0, 777, size=1500).astype(np.int64)
    tt, it = from_oracle(table, "f32"), ids_tensor(ids)
    want = oracle.index_select(table, ids, 0)
    expire_then_recover(cb, lambda st: cb.index_select(tt, it, 0, check=False, status=st), want)


def test_quantised_gather(cb):
    rng = np.random.default_rng(5)
    vocab, hidden = 300, 2048
    qt = make_qtable(rng, "q4_0", vocab, hidden)
    ids = rng.integers(0, vocab, size=900).astype(np.uint32)
    q = cb.QTensor.from_raw(torch.from_numpy(qt), cb.GgmlDType.Q4_0, (vocab, hidden), device="cuda")
    it = ids_tensor(ids)
    want = oracle.qembedding(qt, "q4_0", ids, "f16")
    expire_then_recover(cb, lambda st: q.embedding(it, torch.float16, check=False, status=st), want)


def test_kquant_lookup_norm(cb):
    from helpers import make_kq_blocks

    rng = np.random.default_rng(6)
    vocab, hidden = 256, 4096
    raw = make_kq_blocks(rng, "q4k", vocab * hidden // 256).reshape(vocab, -1)
    ids = rng.integers(0, vocab, size=1500).astype(np.uint32)
    alpha = randn(rng, (hidden,), "bf16", 1.0, 0.1)
    q = cb.QTensor.from_raw(torch.from_numpy(raw), cb.GgmlDType.Q4K, (vocab, hidden), device="cuda")
    it, at = ids_tensor(ids), from_oracle(alpha, "bf16")
    want = oracle.rms_norm(oracle.qembedding(raw, "q4k", ids, "bf16"), alpha, 1e-5, "bf16")
    expire_then_recover(cb, lambda st: cb.qembedding_rms_norm(q, it, at, 1e-5, check=False, status=st), want)
