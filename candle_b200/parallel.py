"""One-process-per-GPU partitioning of the path.

Token rows are independent for every op here, so the default is to give each rank a contiguous
block of rows with the table and the norm weights replicated and no collective at all
(``row_shard``).  The exception is a vocabulary-sharded table (the way candle's sharded loader
splits dim 0, candle-nn/src/var_builder.rs:687-715): every rank looks all ids up in its slice of
the table, writes rows it does not own as zero bits, and one NCCL sum over NVLink assembles the
rows.  The sum runs over the BIT PATTERNS taken as unsigned integers: each element has a single
non-zero contributor, so its bits come through whatever they encode (-0.0, subnormals, NaN
payloads), which a floating-point sum does not promise.  The collective mirrors the only one candle has,
``AllReduce: CustomOp1`` around ``Comm::all_reduce`` in
candle-examples/examples/llama_multiprocess/model.rs:31-90.

torch.distributed is used for the process group and the NCCL call only.
"""
from __future__ import annotations

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


def as_words(t: torch.Tensor) -> torch.Tensor:
    """A contiguous tensor's storage as a flat integer tensor (32-bit words when the byte count
    allows, bytes otherwise): what the shards' partial rows are summed as."""
    if not t.is_contiguous():
        raise CandleError("the rows to be summed over the ranks must be contiguous")
    flat = t.reshape(-1)
    nbytes = flat.numel() * flat.element_size()
    return flat.view(torch.int32) if nbytes % 4 == 0 else flat.view(torch.uint8)


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
            dist.all_reduce(as_words(part), op=dist.ReduceOp.SUM, group=self.group)
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
            dist.all_reduce(as_words(flat), op=dist.ReduceOp.SUM, group=self.group)
            return ops.rms_norm(flat, alpha, eps).reshape(part.shape)
        rows = flat.shape[0]
        if rows % self.world != 0:
            raise CandleError(f"reduce-scatter needs the {rows} token rows to divide by the world size {self.world}")
        mine = torch.empty(rows // self.world, hidden, dtype=flat.dtype, device=flat.device)
        dist.reduce_scatter_tensor(as_words(mine), as_words(flat), op=dist.ReduceOp.SUM, group=self.group)
        return ops.rms_norm(mine, alpha, eps)

    def forward_rms_norm_owner(self, ids: torch.Tensor, alpha: torch.Tensor, eps: float, dst_ptrs, *,
                               status: torch.Tensor | None = None) -> None:
        """The exchange fused into the lookup: this rank decodes and normalises only the ids it owns
        and stores each finished row into every rank's buffer (``dst_ptrs`` from
        ``peer_mapped_empty``), so the rows cross NVLink once, already normalised, and nothing is
        summed.  The buffers are complete once all ranks have passed a barrier after the call.

        Reuse rule: a peer may still be reading a buffer when the fastest rank starts its next step,
        and that step's stores go straight into the peers' memory.  Alternate two buffers per rank,
        or put a second barrier after the readers are done, before calling again with the same one."""
        ops.qembedding_rms_norm_owner(self.table, ids, alpha, eps, dst_ptrs, vocab_range=(self.begin, self.end),
                                      vocab=self.vocab, status=status)

    def forward_rms_norm_row_owner(self, ids: torch.Tensor, alpha: torch.Tensor, eps: float, dst_ptrs_by_rank, *,
                                   status: torch.Tensor | None = None) -> tuple[int, int]:
        """For callers that continue row-sharded: each finished row goes only to the rank whose
        ``row_shard`` of the token rows contains it (``dst_ptrs_by_rank`` from
        ``peer_mapped_empty(..., rank_order=True)`` with buffers of ``row_shard`` size), so about
        (N-1)/N^2 of the output leaves each GPU.  Returns this rank's ``(begin, end)`` rows; its
        buffer holds them once all ranks have passed a barrier.  Same reuse rule as
        ``forward_rms_norm_owner``."""
        rows = ids.numel()
        bounds = [row_shard(rows, r, self.world)[0] for r in range(self.world)] + [rows]
        ops.qembedding_rms_norm_row_owner(self.table, ids, alpha, eps, dst_ptrs_by_rank, bounds,
                                          vocab_range=(self.begin, self.end), vocab=self.vocab, status=status)
        return bounds[self.rank], bounds[self.rank + 1]


class RoutedQEmbedding:
    """Vocabulary-sharded table, row-sharded consumers, exchange in QUANTISED form: each rank routes the
    raw block rows of the ids it owns to the rank whose ``row_shard`` of the token rows holds them
    (``cb200_qembedding_route_rows``), the ranks meet at a barrier, and every rank decodes and
    normalises its own block locally.  Two staging buffers per rank alternate, so the stores of step
    i + 1 never land in rows a rank still decodes from step i."""

    def __init__(self, sharded: ShardedQEmbedding, max_rows: int, group=None):
        self.emb, self.group = sharded, group
        self.block_rows = -(-max_rows // sharded.world)
        row_bytes = sharded.table.shape[1] // sharded.table.dtype.block_size * sharded.table.dtype.type_size
        dev = sharded.table.data.device
        self.staging = [peer_mapped_empty((self.block_rows, row_bytes), torch.uint8, dev, group, rank_order=True)
                        for _ in range(2)]
        self.iota = torch.arange(self.block_rows, dtype=torch.int32, device=dev)
        self.flag = torch.zeros(1, device=dev)
        self.step = 0

    def forward_rms_norm(self, ids: torch.Tensor, alpha: torch.Tensor, eps: float, *, status=None) -> torch.Tensor:
        """Returns this rank's ``row_shard`` of ``rms_norm(lookup(ids))`` as ``[rows_r, hidden]``."""
        import torch.distributed as dist

        e = self.emb
        rows = ids.numel()
        if -(-rows // e.world) > self.block_rows:
            raise CandleError(f"{rows} token rows exceed the staging buffers of {self.block_rows} rows per rank")
        bounds = [row_shard(rows, r, e.world)[0] for r in range(e.world)] + [rows]
        local, ptrs = self.staging[self.step & 1]
        self.step += 1
        ops.qembedding_route_rows(e.table, ids, ptrs, bounds, vocab_range=(e.begin, e.end), vocab=e.vocab, status=status)
        dist.all_reduce(self.flag, group=self.group)  # the ranks' barrier, in stream order
        mine = bounds[e.rank + 1] - bounds[e.rank]
        staged = QTensor(local[:mine].reshape(-1), e.table.dtype, (mine, e.table.shape[1]))
        return ops.qembedding_rms_norm(staged, self.iota[:mine], alpha, eps, check=False, status=status)


def peer_mapped_empty(shape, dtype: torch.dtype, device, group=None, rank_order: bool = False):
    """A buffer of ``shape`` on every rank of ``group`` (the same shape everywhere), each one mapped
    into every rank's address space (torch's symmetric memory: CUDA virtual-memory handles exchanged
    over the process group).  Returns ``(local tensor, device addresses of all ranks' buffers)``, this
    rank's own first -- the destination list ``ShardedQEmbedding.forward_rms_norm_owner`` takes -- or
    in rank order with ``rank_order=True`` (what ``forward_rms_norm_row_owner`` takes).  NVLink
    multicast is switched off: only plain peer stores go through these mappings.  Contents written by
    peers are visible after a barrier between the ranks; see the reuse rule of
    ``forward_rms_norm_owner``."""
    import os

    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm

    g = group if group is not None else dist.group.WORLD
    t = symm.empty(*shape, dtype=dtype, device=device)
    hdl = symm.rendezvous(t, g.group_name)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    if rank_order:
        return t, ptrs
    mine = hdl.rank
    return t, [ptrs[mine]] + [p for i, p in enumerate(ptrs) if i != mine]
