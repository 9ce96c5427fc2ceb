"""World-size-2 (and 4) CPU runs over gloo of the vocab-sharded path.

``test_masked_partials_sum_to_unsharded_lookup``: the algebra -- every rank decodes the ids it owns,
writes zero bits elsewhere, and the sum of the bit patterns over ranks equals the unsharded lookup bit
for bit (-0.0 included).
``test_sharded_embedding_host_logic``: the library's own ``ShardedQEmbedding`` driven over gloo --
shard arithmetic, the all-reduce and the reduce-scatter route with its row split, reshapes and error
cases.  There is no GPU here, so the two device steps the class calls (the masked lookup of its table
and ``ops.rms_norm``) are replaced by CPU stand-ins that compute the same thing with the oracle;
everything between them is the product code.  The GPU kernels themselves are compared against the
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
        part = np.zeros((n, hidden), dtype=np.uint16)  # foreign rows: zero bits
        if owned.any():
            part[owned] = oracle.qembedding(qt[begin:end], qtype, (ids[owned] - begin).astype(np.uint32), "bf16")
        # the sum over ranks runs on the bit patterns as 32-bit integers, as the product's collective does:
        # each word has one non-zero contributor
        t = torch.from_numpy(part.view(np.int32).copy())
        dist.all_reduce(t)
        total = t.numpy().view(np.uint16).reshape(n, hidden)
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


class _CpuTable:
    """Stand-in for a QTensor shard: same ``shape`` and ``embedding`` contract, values from the oracle."""

    def __init__(self, qt_local, qtype, hidden):
        self.qt, self.qtype, self.shape = qt_local, qtype, (qt_local.shape[0], hidden)

    def embedding(self, ids, dtype, *, check=True, status=None, vocab_range=None, vocab=None):
        import oracle

        assert dtype == torch.bfloat16 and vocab_range is not None and vocab_range[1] - vocab_range[0] == self.shape[0]
        flat = ids.reshape(-1).numpy().astype(np.uint32)
        assert flat.max() < vocab
        begin, end = vocab_range
        owned = (flat >= begin) & (flat < end)
        part = np.zeros((flat.size, self.shape[1]), dtype=np.uint16)
        if owned.any():
            part[owned] = oracle.qembedding(self.qt, self.qtype, (flat[owned] - begin).astype(np.uint32), "bf16")
        return torch.from_numpy(part.view(np.int16)).view(torch.bfloat16).reshape(tuple(ids.shape) + (self.shape[1],))


def _host_logic_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from candle_b200 import CandleError, parallel
        from helpers import make_qtable

        def cpu_rms_norm(x, alpha, eps):  # stands in for the CUDA op on this GPU-less host
            xo = x.contiguous().view(torch.int16).numpy().view(np.uint16)
            ao = alpha.view(torch.int16).numpy().view(np.uint16)
            return torch.from_numpy(oracle.rms_norm(xo, ao, eps, "bf16").view(np.int16)).view(torch.bfloat16)

        parallel.ops.rms_norm = cpu_rms_norm
        rng = np.random.default_rng(19)
        vocab, hidden = 32 * world, 128
        qt = make_qtable(rng, "q4_0", vocab, hidden)
        qt[:, :2] = 0
        alpha_np = oracle.cast_from_f32((1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32), "bf16")
        alpha = torch.from_numpy(alpha_np.view(np.int16)).view(torch.bfloat16)
        ids_np = rng.integers(0, vocab, size=(4, 3 * world)).astype(np.int64)
        ids = torch.from_numpy(ids_np)
        b, e = parallel.vocab_shard(vocab, rank, world)
        emb = parallel.ShardedQEmbedding(_CpuTable(qt[b:e], "q4_0", hidden), vocab, rank, world, torch.bfloat16)
        want_rows = oracle.qembedding(qt, "q4_0", ids_np, "bf16")
        want = oracle.rms_norm(want_rows, alpha_np, 1e-5, "bf16")
        bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
        ok = (emb.begin, emb.end) == (b, e)
        rows = emb.forward(ids)
        ok = ok and tuple(rows.shape) == (4, 3 * world, hidden) and np.array_equal(bits(rows), want_rows)
        y = emb.forward_rms_norm(ids, alpha, 1e-5)
        ok = ok and tuple(y.shape) == (4, 3 * world, hidden) and np.array_equal(bits(y), want)
        ys = emb.forward_rms_norm(ids, alpha, 1e-5, scatter=True)
        rb, re = parallel.row_shard(ids.numel(), rank, world)
        ok = ok and tuple(ys.shape) == (re - rb, hidden) and np.array_equal(bits(ys), want.reshape(-1, hidden)[rb:re])
        # the reduce-scatter route needs the token rows to divide by the world size
        try:
            emb.forward_rms_norm(ids.reshape(-1)[: ids.numel() - 1], alpha, 1e-5, scatter=True)
            ok = False
        except CandleError as exc:
            ok = ok and "divide by the world size" in str(exc)
        # a shard of the wrong size is refused at construction
        try:
            parallel.ShardedQEmbedding(_CpuTable(qt[b:e - 1], "q4_0", hidden), vocab, rank, world)
            ok = False
        except CandleError as exc:
            ok = ok and "table rows" in str(exc)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_embedding_host_logic(world):
    import oracle

    oracle.build()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_host_logic_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_as_words_views_the_same_storage():
    # what the ranks' partial rows are summed as: 32-bit words over the same bytes (bytes for an odd
    # number of 16-bit values); a non-contiguous tensor is refused instead of being copied silently
    from candle_b200 import CandleError
    from candle_b200.parallel import as_words

    t = torch.arange(12, dtype=torch.float32).to(torch.bfloat16).reshape(3, 4)
    w = as_words(t)
    assert w.dtype == torch.int32 and w.numel() == 6 and w.data_ptr() == t.data_ptr()
    w += w  # doubling the words in place is visible through the original tensor's storage
    assert t.view(torch.int16).reshape(-1)[1].item() == 2 * torch.tensor(1.0).to(torch.bfloat16).view(torch.int16).item()
    odd = torch.zeros(3, dtype=torch.float16)
    assert as_words(odd).dtype == torch.uint8 and as_words(odd).numel() == 6
    with pytest.raises(CandleError):
        as_words(t.t())
