"""Communicator set-up with a deadline (``cb200_nccl_comm_init_timeout``): the failure is made on the
host -- a rank that never joins -- and no device work is involved.  candle's own set-up waits for a
missing peer for ever (candle-examples/examples/llama_multiprocess/main.rs:156-158)."""
import time

import numpy as np
import pytest
import torch

import oracle
from helpers import from_oracle, ids_tensor, make_qtable, randn, to_oracle

pytestmark = pytest.mark.gpu


def test_init_with_deadline_single_rank_then_sharded_call(cb):
    # all ranks present (there is one): the non-blocking communicator works with the sharded entry point
    from candle_b200 import _nccl
    from candle_b200.ops import _stream, new_status, raise_for_status

    rng = np.random.default_rng(71)
    vocab, hidden, n = 200, 4096, 500
    comm = _nccl.comm_init_timeout(1, _nccl.unique_id(), 0, 60_000)
    try:
        qt = make_qtable(rng, "q8_0", vocab, hidden)
        ids = rng.integers(0, vocab, size=(n,)).astype(np.uint32)
        alpha = randn(rng, (hidden,), "bf16", 1.0, 0.1)
        want = oracle.rms_norm(oracle.qembedding(qt, "q8_0", ids, "bf16"), alpha, 1e-5, "bf16")
        tq, tids, ta = torch.from_numpy(qt).cuda(), ids_tensor(ids), from_oracle(alpha, "bf16")
        y = torch.empty(n, hidden, dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(n, hidden, dtype=torch.bfloat16, device="cuda")
        st = new_status("cuda")
        _nccl.call("cb200_sharded_qembedding_rms_norm", comm, tq.data_ptr(), 8, tids.data_ptr(), ta.data_ptr(),
                   y.data_ptr(), scratch.data_ptr(), scratch.numel() * 2, vocab, hidden, n, 1e-5, 2, 1, 0, vocab, 0,
                   st.data_ptr(), _stream(y))
        raise_for_status(st)
        assert np.array_equal(to_oracle(y), want)
    finally:
        torch.cuda.synchronize()
        _nccl.comm_destroy(comm)


def test_missing_peer_ends_in_a_timeout_not_a_hang(cb):
    # a two-rank communicator whose second rank never calls: the call returns E_TIMEOUT after the
    # deadline, leaves no communicator behind, and the device goes on working
    from candle_b200 import _cabi, _nccl

    t0 = time.monotonic()
    with pytest.raises(_cabi.CandleB200Error) as err:
        _nccl.comm_init_timeout(2, _nccl.unique_id(), 0, 1500)
    waited = time.monotonic() - t0
    assert err.value.code == _nccl.E_TIMEOUT
    assert 1.0 <= waited < 30.0, waited
    x = torch.randn(64, 1024, device="cuda").to(torch.bfloat16)
    alpha = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    y = cb.rms_norm(x, alpha, 1e-5)
    assert np.array_equal(to_oracle(y), oracle.rms_norm(to_oracle(x), to_oracle(alpha), 1e-5, "bf16"))


def test_bad_arguments_are_refused_on_the_host(cb):
    from candle_b200 import _nccl
    import ctypes

    comm = ctypes.c_void_p()
    uid = ctypes.create_string_buffer(_nccl.unique_id(), _nccl.UNIQUE_ID_BYTES)
    f = _nccl.lib.cb200_nccl_comm_init_timeout
    assert f(ctypes.byref(comm), 2, ctypes.cast(uid, ctypes.c_void_p), 2, 100) == -1   # rank out of range
    assert f(ctypes.byref(comm), 0, ctypes.cast(uid, ctypes.c_void_p), 0, 100) == -1   # no ranks
    assert f(ctypes.byref(comm), 1, ctypes.cast(uid, ctypes.c_void_p), 0, -5) == -1    # negative deadline
    assert f(None, 1, ctypes.cast(uid, ctypes.c_void_p), 0, 100) == -1
