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

    def forward_rms_norm_owner(self, ids: torch.Tensor, alpha: torch.Tensor, eps: float, dst_ptrs, *,
                               status: torch.Tensor | None = None) -> None:
        """The exchange fused into the lookup: this rank decodes and normalises only the ids it owns
        and stores each finished row into every rank's buffer (``dst_ptrs`` from
        ``peer_mapped_empty``), so the rows cross NVLink once, already normalised, and nothing is
        summed.  The buffers are complete once all ranks have passed a barrier after the call."""
        ops.qembedding_rms_norm_owner(self.table, ids, alpha, eps, dst_ptrs, vocab_range=(self.begin, self.end),
                                      vocab=self.vocab, status=status)


def peer_mapped_empty(shape, dtype: torch.dtype, device, group=None):
    """A buffer of ``shape`` on every rank of ``group``, each one mapped into every rank's address
    space (torch's symmetric memory: CUDA virtual-memory handles exchanged over the process group).
    Returns ``(local tensor, device addresses of all ranks' buffers with this rank's own first)`` --
    the destination list ``ShardedQEmbedding.forward_rms_norm_owner`` takes.  NVLink multicast is
    switched off: only plain peer stores go through these mappings."""
    import os

    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm

    g = group if group is not None else dist.group.WORLD
    t = symm.empty(*shape, dtype=dtype, device=device)
    hdl = symm.rendezvous(t, g.group_name)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    mine = hdl.rank
    return t, [ptrs[mine]] + [p for i, p in enumerate(ptrs) if i != mine]


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
    # owner-writes-to-all variant: lookup + norm of the owned rows, stored into every rank's buffer
    owner = None
    try:
        shared, dsts = peer_mapped_empty((wl.rows, wl.hidden), torch.bfloat16, dev)
        flag = torch.zeros(1, device=dev)

        def owner_step(i):
            emb.forward_rms_norm_owner(ids[i % 2], alpha, wl.eps, dsts, status=st)
            dist.all_reduce(flag)  # the ranks' barrier, in stream order: all rows have landed after it

        owner_step(0)
        torch.cuda.synchronize()
        owner_ok = bool(np.array_equal(to_oracle(shared[:256]), want)) and int(st[0].item()) == 0
        k = max(2, steps // 2)
        ms_owner = timed(owner_step, k, 2) / k
        owner = {"ms_per_step": ms_owner, "tokens_per_s": wl.rows / (ms_owner * 1e-3),
                 "nvlink_out_gbs_per_gpu": (world - 1) / world * wl.rows * wl.hidden * 2 / (ms_owner * 1e-3) / 1e9,
                 "parity": "bit-exact vs unsharded CPU oracle on the first 256 rows" if owner_ok else "MISMATCH",
                 "note": "each rank decodes + normalises the rows it owns and stores them into every rank's "
                         "buffer (peer stores over NVLink), then one barrier"}
        parity_ok = parity_ok and owner_ok
    except Exception as exc:  # symmetric memory unavailable on this system
        owner = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    # end to end for the owner variant: ids from pinned host memory, this rank's block of the finished rows
    # back to pinned host memory (all ranks together return every row once)
    e2e = None
    if owner is not None and "ms_per_step" in owner:
        rb, re = row_shard(wl.rows, rank, world)
        host_ids = [torch.from_numpy(np.ascontiguousarray(i.reshape(-1)).view(np.int32)).pin_memory() for i in wl.ids]
        dev_ids = torch.empty_like(ids[0].reshape(-1))
        host_out = torch.empty(re - rb, wl.hidden, dtype=torch.bfloat16).pin_memory()

        def e2e_step(i):
            dev_ids.view(torch.uint8).copy_(host_ids[i % 2].view(torch.uint8), non_blocking=True)
            emb.forward_rms_norm_owner(dev_ids, alpha, wl.eps, dsts, status=st)
            dist.all_reduce(flag)
            host_out.copy_(shared[rb:re], non_blocking=True)

        ke = max(2, min(steps, 5))
        ms_e2e = timed(e2e_step, ke, 1) / ke
        e2e = {"value": wl.rows / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": int(dev_ids.numel() * dev_ids.element_size()) * world,
               "d2h_bytes_per_step": wl.rows * wl.hidden * 2,
               "note": "every rank uploads the ids; each rank downloads its 1/N block of the finished rows"}
    if rank == 0:
        peak, kind = measured_peak()
        out_bytes = wl.rows * wl.hidden * 2
        ms_allreduce_step = ms / steps
        use_owner = owner is not None and "ms_per_step" in owner
        ms_per_step = owner["ms_per_step"] if use_owner else ms_allreduce_step
        nvlink_bytes = (world - 1) / world * out_bytes  # leaves each GPU once in the owner variant
        hbm_bytes = (wl.rows * wl.row_qbytes + out_bytes) / world + nvlink_bytes  # owned rows in/out + rows received
        t_hbm, t_link = hbm_bytes / (peak * 1e9), nvlink_bytes / 770e9
        if use_owner:
            roof = {"bound": "nvlink" if t_link >= t_hbm else "hbm",
                    "achieved": nvlink_bytes / (ms_per_step * 1e-3) / 1e9, "peak": 770.0, "unit": "GB/s",
                    "frac": max(t_hbm, t_link) / (ms_per_step * 1e-3), "peak_kind": "of measured",
                    "traffic": None,
                    "note": "fused lookup + norm + exchange: target time = max(HBM bytes / measured HBM peak, "
                            "bytes leaving the GPU / 770 GB/s measured peer-copy bandwidth); frac = target / achieved time"}
        else:
            per_gpu_bytes = wl.rows * wl.row_qbytes / world + out_bytes + 2 * out_bytes
            roof = {"bound": "hbm", "achieved": per_gpu_bytes / (ms_per_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                    "frac": per_gpu_bytes / (ms_per_step * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}", "traffic": None,
                    "note": "per-GPU HBM bytes of lookup + norm over the whole step time, which also contains the "
                            "NVLink all-reduce"}
        print(json.dumps({
            "metric": "tokens/s, embed+norm (HBM GB/s in roofline)", "value": wl.rows / (ms_per_step * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seed 0)",
            "config": {"workload": wl.desc, "rows": wl.rows, "hidden": wl.hidden,
                       "parallelism": (f"vocab sharded x{world}: each rank decodes + normalises the rows it owns and "
                                       "stores them into every rank's buffer over NVLink, one barrier") if use_owner
                       else f"vocab sharded x{world}: masked lookup + NCCL all-reduce + RMSNorm"},
            "owner_writes_variant": owner,
            "all_reduce_variant": {"ms_per_step": ms_allreduce_step, "tokens_per_s": wl.rows / (ms_allreduce_step * 1e-3),
                                   "phases_ms": {"masked_lookup": ms_lookup, "all_reduce": ms_allreduce,
                                                 "rms_norm": ms_norm,
                                                 "all_reduce_busbw_gbs": 2 * (world - 1) / world * out_bytes
                                                 / (ms_allreduce * 1e-3) / 1e9},
                                   "note": "candle's scheme: masked lookup (-0.0 for foreign rows), NCCL sum, norm of "
                                           "every row on every rank"},
            "reduce_scatter_variant": {"ms_per_step": ms_scatter, "tokens_per_s": wl.rows / (ms_scatter * 1e-3),
                                       "note": "sum as reduce-scatter, each rank normalises 1/N of the rows"},
            "roofline": roof, "e2e": e2e, "gpu_launches": steps if use_owner else 2 * steps,
            "parity": "bit-exact vs unsharded CPU oracle on the first 256 rows" if parity_ok else "MISMATCH",
            "clocks": clocks,
        }), flush=True)
    dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit(3)
