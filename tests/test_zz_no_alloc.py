"""The allocation-free entry point, cb200_sharded_qembedding_rms_norm_static, against the entry
point that takes caller scratch.  Some callers cannot call cudaMalloc -- their memory pool already
owns the device, or they sit in a serving loop that cannot afford cudaMalloc's device-wide
synchronisation -- so this variant keeps its intermediate rows in an array built into the library.
Called through the C ABI, twice in a row (the array is shared by all calls and keeps old contents),
and compared bit for bit with the caller-scratch entry and with the CPU oracle; the second call must
leave the device's free memory exactly as it found it.  This file is collected last on purpose."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_caller_scratch_entry():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from candle_b200 import _nccl
    from candle_b200.ops import _stream, new_status
    from helpers import ids_tensor, make_qtable, randn, from_oracle, to_oracle
    import oracle

    rng = np.random.default_rng(53)
    vocab, hidden = 500, 4096
    alpha_np = randn(rng, (hidden,), "bf16", 1.0, 0.1)
    alpha = from_oracle(alpha_np, "bf16")
    stream = _stream(alpha)
    for call_no, (qtype, code, n) in enumerate((("q8_0", 8, 3000), ("q4_0", 2, 1234))):
        # second call: different table, fewer rows -> stale rows of the first call stay in the array
        qt_np = make_qtable(rng, qtype, vocab, hidden)
        ids_np = rng.integers(0, vocab, size=(n,)).astype(np.uint32)
        qt, ids = torch.from_numpy(qt_np).cuda(), ids_tensor(ids_np)
        y_ref = torch.empty(n, hidden, dtype=torch.bfloat16, device="cuda")
        y_new = torch.full((n, hidden), 7.0, dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(n, hidden, dtype=torch.bfloat16, device="cuda")
        st = new_status("cuda")
        # comm = NULL: single rank, no NCCL call at all
        _nccl.call("cb200_sharded_qembedding_rms_norm", None, qt.data_ptr(), code, ids.data_ptr(), alpha.data_ptr(),
                   y_ref.data_ptr(), scratch.data_ptr(), scratch.numel() * 2, vocab, hidden, n, 1e-5, 2, 1, 0, vocab, 0,
                   st.data_ptr(), stream)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _nccl.call("cb200_sharded_qembedding_rms_norm_static", None, qt.data_ptr(), code, ids.data_ptr(),
                   alpha.data_ptr(), y_new.data_ptr(), vocab, hidden, n, 1e-5, 2, 1, 0, vocab, 0, st.data_ptr(), stream)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        assert st[0].item() == 0
        assert torch.equal(y_new.view(torch.int16), y_ref.view(torch.int16)), f"call {call_no} differs"
        want = oracle.rms_norm(oracle.qembedding(qt_np, qtype, ids_np, "bf16"), alpha_np, 1e-5, "bf16")
        assert np.array_equal(to_oracle(y_new), want), f"call {call_no} differs from the CPU oracle"
        if call_no > 0:  # the first call on a device may load the library's device image, array included
            assert free_after == free_before, "the allocation-free entry changed the device's free memory"
    # a request beyond the built-in array is refused on the host, nothing is launched
    too_many = _nccl.STATIC_SCRATCH_BYTES // (hidden * 2) + 1
    rc = _nccl.lib.cb200_sharded_qembedding_rms_norm_static(None, qt.data_ptr(), 2, ids.data_ptr(), alpha.data_ptr(),
                                                            y_new.data_ptr(), vocab, hidden, too_many, 1e-5, 2, 1, 0,
                                                            vocab, 0, None, stream)
    assert rc == -5
