"""One-process-per-GPU partitioning of the path.

Token rows are independent for every op here, so the default is to give each rank a contiguous
block of rows with the table and the norm weights replicated and no collective at all
(``row_shard``).  The exception is a vocabulary-sharded table (the way candle's sharded loader
splits dim 0, candle-nn/src/var_builder.rs:687-715): every rank looks all ids up in its slice of
the table, writes rows it does not own as -0.0 -- the additive identity that also preserves a
-0.0 coming from the owner -- and one NCCL sum over NVLink assembles the rows, exactly, because
each element has a single non-zero contributor.  The collective mirrors the only one candle has,
``AllReduce: CustomOp1`` around ``Comm::all_reduce`` in
candle-examples/examples/llama_multiprocess/model.rs:31-90.

torch.distributed is used for the process group and the NCCL call only.
"""
from __future__ import annotations

import json

import torch

from . import ops
from .errors import CandleError
from .quantized import QTensor


def row_shard(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [begin, end) of rank ``rank``: contiguous blocks, sizes differing by at most one."""
    if not 0 <= rank < world:
        raise CandleError(f"rank {rank} outside world of {world}")
    base, extra = divmod(rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def vocab_shard(vocab: int, rank: int, world: int) -> tuple[int, int]:
    """Vocabulary rows [begin, end) of rank ``rank``; the table's dim 0 must divide evenly, as
    candle's ``ShardedSafeTensors`` requires (candle-nn/src/var_builder.rs:700-703)."""
    if not 0 <= rank < world:
        raise CandleError(f"rank {rank} outside world of {world}")
    if vocab % world != 0:
        raise CandleError(f"The size in dim 0 ({vocab}) is not divisible by the world size ({world})")
    per = vocab // world
    return rank * per, (rank + 1) * per


class ShardedQEmbedding:
    """A Q4_0 / Q8_0 table split by vocabulary over the ranks of ``group``.

    ``forward(ids)`` returns the full ``ids.shape + [hidden]`` rows on every rank (masked lookup +
    all-reduce); ``forward_rms_norm`` also applies the RMS norm.  With ``scatter=True`` the sum is
    a reduce-scatter instead and each rank normalises and returns only its ``row_shard`` of the
    token rows -- 1/N of the norm traffic, for callers that continue row-sharded."""

    def __init__(self, local_table: QTensor, vocab: int, rank: int, world: int, dtype: torch.dtype = torch.bfloat16,
                 group=None):
        self.table, self.vocab, self.rank, self.world, self.dtype, self.group = local_table, vocab, rank, world, dtype, group
        self.begin, self.end = vocab_shard(vocab, rank, world)
        if local_table.shape[0] != self.end - self.begin:
            raise CandleError(f"rank {rank} expects {self.end - self.begin} table rows, got {local_table.shape[0]}")

    def partial(self, ids: torch.Tensor, *, check: bool = True, status=None) -> torch.Tensor:
        return self.table.embedding(ids, self.dtype, check=check, status=status,
                                    vocab_range=(self.begin, self.end), vocab=self.vocab)

    def forward(self, ids: torch.Tensor, *, check: bool = True) -> torch.Tensor:
        import torch.distributed as dist

        part = self.partial(ids, check=check)
        if self.world > 1:
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
        return part

    def forward_rms_norm(self, ids: torch.Tensor, alpha: torch.Tensor, eps: float, *, scatter: bool = False,
                         check: bool = True) -> torch.Tensor:
        import torch.distributed as dist

        part = self.partial(ids, check=check)
        hidden = part.shape[-1]
        flat = part.reshape(-1, hidden)
        if self.world == 1:
            return ops.rms_norm(flat, alpha, eps).reshape(part.shape)
        if not scatter:
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
            return ops.rms_norm(flat, alpha, eps).reshape(part.shape)
        rows = flat.shape[0]
        if rows % self.world != 0:
            raise CandleError(f"reduce-scatter needs the {rows} token rows to divide by the world size {self.world}")
        mine = torch.empty(rows // self.world, hidden, dtype=flat.dtype, device=flat.device)
        dist.reduce_scatter_tensor(mine, flat, op=dist.ReduceOp.SUM, group=self.group)
        return ops.rms_norm(mine, alpha, eps)


def bench_c4(args, rank: int, world: int, dev) -> None:
    """The vocab-sharded benchmark configuration (called by bench.py with the process group up)."""
    import os
    import sys

    import numpy as np
    import torch.distributed as dist

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from bench import ClockSampler, Workload, measured_peak  # noqa: E402
    from helpers import from_oracle, ids_tensor, to_oracle  # noqa: E402
    import oracle  # noqa: E402

    from .quantized import GgmlDType

    if world < 2:
        raise SystemExit("the vocab-sharded C4 workload needs --gpus >= 2 (launch with torch.distributed.run)")
    wl = Workload("c4", args.rows_scale)
    begin, end = vocab_shard(wl.vocab, rank, world)
    local = QTensor.from_raw(torch.from_numpy(wl.qtable[begin:end]), GgmlDType.Q4_0, (end - begin, wl.hidden), device=dev)
    emb = ShardedQEmbedding(local, wl.vocab, rank, world, torch.bfloat16)
    alpha = from_oracle(wl.alpha, "bf16", dev)
    ids = [ids_tensor(i, dev) for i in wl.ids]
    stream = torch.cuda.current_stream()
    st = ops.new_status(dev)

    y = emb.forward_rms_norm(ids[0], alpha, wl.eps)
    torch.cuda.synchronize()
    sample = wl.ids[0][:256]
    want = oracle.rms_norm(oracle.qembedding(wl.qtable, wl.qtype, sample, "bf16"), wl.alpha, wl.eps, "bf16")
    parity_ok = bool(np.array_equal(to_oracle(y[:256]), want))
    del y

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(warmup + i)
        e1.record(stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    steps = args.steps
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    ms = timed(lambda i: emb.forward_rms_norm(ids[i % 2], alpha, wl.eps, check=False), steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    ms_scatter = timed(lambda i: emb.forward_rms_norm(ids[i % 2], alpha, wl.eps, scatter=True, check=False),
                       max(2, steps // 2), 2) / max(2, steps // 2)
    # phases, timed separately
    ms_lookup = timed(lambda i: emb.partial(ids[i % 2], check=False, status=st), 5, 2) / 5
    buf = emb.partial(ids[0], check=False, status=st).reshape(-1, wl.hidden)
    ms_allreduce = timed(lambda i: dist.all_reduce(buf), 5, 2) / 5
    ms_norm = timed(lambda i: ops.rms_norm(buf, alpha, wl.eps), 5, 2) / 5
    if rank == 0:
        peak, kind = measured_peak()
        out_bytes = wl.rows * wl.hidden * 2
        per_gpu_bytes = wl.rows * wl.row_qbytes / world + out_bytes + 2 * out_bytes  # lookup + norm; all-reduce is NVLink
        ms_per_step = ms / steps
        print(json.dumps({
            "metric": "tokens/s, embed+norm (HBM GB/s in roofline)", "value": wl.rows / (ms_per_step * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seed 0)",
            "config": {"workload": wl.desc, "rows": wl.rows, "hidden": wl.hidden,
                       "parallelism": f"vocab sharded x{world}: masked lookup + NCCL all-reduce + RMSNorm"},
            "phases_ms": {"masked_lookup": ms_lookup, "all_reduce": ms_allreduce, "rms_norm": ms_norm,
                          "all_reduce_busbw_gbs": 2 * (world - 1) / world * out_bytes / (ms_allreduce * 1e-3) / 1e9},
            "reduce_scatter_variant": {"ms_per_step": ms_scatter, "tokens_per_s": wl.rows / (ms_scatter * 1e-3),
                                       "note": "sum as reduce-scatter, each rank normalises 1/N of the rows"},
            "roofline": {"bound": "hbm", "achieved": per_gpu_bytes / (ms_per_step * 1e-3) / 1e9, "peak": peak,
                         "unit": "GB/s", "frac": per_gpu_bytes / (ms_per_step * 1e-3) / 1e9 / peak,
                         "peak_kind": f"of {kind}", "traffic": None,
                         "note": "per-GPU HBM bytes of lookup + norm over the whole step time, which also contains "
                                 "the NVLink all-reduce"},
            "e2e": None, "gpu_launches": 2 * steps,
            "parity": "bit-exact vs unsharded CPU oracle on the first 256 rows" if parity_ok else "MISMATCH",
            "clocks": clocks,
        }), flush=True)
    dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit(3)
