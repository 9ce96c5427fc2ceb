"""World-size-2 (and 4) CPU runs over gloo of the vocab-sharded algebra: every rank decodes the ids
it owns, writes -0.0 elsewhere, and the sum over ranks must equal the unsharded lookup bit for bit.
The per-rank partials come from the CPU oracle here; the GPU kernels are compared against the same
oracle in the gpu tests."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, qtype, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from candle_b200.parallel import row_shard, vocab_shard
        from helpers import make_qtable

        rng = np.random.default_rng(7)  # same stream on every rank: replicated ids, full table
        vocab, hidden, n = 64 * world, 256, 200
        qt = make_qtable(rng, qtype, vocab, hidden)
        qt[:, :2] = 0  # first block of every row has scale +0: -0.0 / +0.0 values appear
        ids = rng.integers(0, vocab, size=n).astype(np.uint32)
        begin, end = vocab_shard(vocab, rank, world)
        owned = (ids >= begin) & (ids < end)
        part = np.full((n, hidden), 0x8000, dtype=np.uint16)  # bf16 -0.0
        if owned.any():
            part[owned] = oracle.qembedding(qt[begin:end], qtype, (ids[owned] - begin).astype(np.uint32), "bf16")
        # bf16 sum over ranks; each element has one non-zero contributor, so summing in f32 and
        # rounding back is the exact bf16 sum NCCL computes
        t = torch.from_numpy(part.view(np.int16)).view(torch.bfloat16).to(torch.float32)
        dist.all_reduce(t)
        total = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
        want = oracle.qembedding(qt, qtype, ids, "bf16")
        ok = np.array_equal(total, want)
        # the row-sharded continuation: each rank normalises its block of rows; together = unsharded
        a = oracle.cast_from_f32((1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32), "bf16")
        b, e = row_shard(n, rank, world)
        mine = oracle.rms_norm(total[b:e], a, 1e-5, "bf16")
        ok = ok and np.array_equal(mine, oracle.rms_norm(want, a, 1e-5, "bf16")[b:e])
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("qtype", ["q8_0", "q4_0"])
@pytest.mark.parametrize("world", [2, 4])
def test_masked_partials_sum_to_unsharded_lookup(world, qtype):
    import oracle

    oracle.build()
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, qtype, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
