"""Batch-dimension (and, for small batches, column) sharding of lm2exp / lt2exp across the GPUs of one node.

Every batch entry r of both ops is independent (the reference's kernels only use the batch index to offset
pointers, triturus/lm2exp.py:94,122-123 and triturus/lt2exp.py:264,301-303), so the multi-GPU path is one
process per GPU, each owning a contiguous block of r, with no collective on the data path.  The only
communication offered is an optional all-gather of the output shards (`gather_batch`), which callers time
and report separately.  The K columns are independent too (one stabiliser per (r, k)), so a batch with fewer
entries than there are ranks is cut along k instead, with the first operand replicated (`shard_columns`,
`gather_columns`); there is still no exchange on the data path.  Works with the NCCL backend on GPUs and the
gloo backend on CPU tensors.
"""

from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist


def shard_bounds(batch: int, rank: int, world_size: int) -> tuple[int, int]:
    """Contiguous block [lo, hi) of the batch owned by `rank`; the first `batch % world_size` ranks get
    one extra entry, ranks beyond the batch get an empty block."""
    if batch < 0 or world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad sharding request: batch={batch} rank={rank} world_size={world_size}")
    base, extra = divmod(batch, world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo, hi


def shard_batch(tensors: Sequence[torch.Tensor], rank: int, world_size: int) -> tuple[torch.Tensor, ...]:
    """Slice dim 0 of every tensor to this rank's block (views, no copy)."""
    batch = tensors[0].shape[0]
    if any(t.shape[0] != batch for t in tensors):
        raise ValueError("all operands must share the batch dimension")
    lo, hi = shard_bounds(batch, rank, world_size)
    return tuple(t[lo:hi] for t in tensors)


def gather_batch(shard: torch.Tensor, batch: int, group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """All-gather output shards along dim 0 into the full [batch, ...] result on every rank.

    Equal shards use a single `all_gather_into_tensor`; ragged shards (batch not divisible by the world
    size) are padded to the largest shard first.
    """
    world = dist.get_world_size(group)
    sizes = [hi - lo for lo, hi in (shard_bounds(batch, r, world) for r in range(world))]
    if shard.shape[0] != sizes[dist.get_rank(group)]:
        raise ValueError(f"shard has {shard.shape[0]} batch entries, expected {sizes[dist.get_rank(group)]}")
    biggest = max(sizes)
    tail = tuple(shard.shape[1:])
    if biggest == 0:
        return shard.new_empty((0, *tail))
    if shard.shape[0] != biggest:
        padded = shard.new_zeros((biggest, *tail))
        padded[: shard.shape[0]] = shard
    else:
        padded = shard.contiguous()
    full = shard.new_empty((world * biggest, *tail))
    dist.all_gather_into_tensor(full, padded, group=group)
    if all(s == biggest for s in sizes):
        return full
    parts = [full[r * biggest : r * biggest + sizes[r]] for r in range(world)]
    return torch.cat(parts, dim=0)


def column_bounds(columns: int, rank: int, world_size: int) -> tuple[int, int]:
    """Contiguous block [lo, hi) of the K columns owned by `rank`.  The stabiliser is per (r, k) column, so
    columns are as independent as batch entries.  When K is a multiple of 4 the cuts fall on multiples of 4,
    which keeps every slice of b 16-byte aligned for TMA (no padded copy)."""
    unit = 4 if columns % 4 == 0 else 1
    lo, hi = shard_bounds(columns // unit, rank, world_size)
    return lo * unit, hi * unit


def shard_columns(tensors: Sequence[torch.Tensor], rank: int, world_size: int) -> tuple[torch.Tensor, ...]:
    """Column sharding: the first operand (a of lm2exp, w of lt2exp) is replicated, every other operand is
    sliced along its last dimension k to this rank's block (views, no copy)."""
    columns = tensors[-1].shape[-1]
    if any(t.shape[-1] != columns for t in tensors[1:]):
        raise ValueError("all log-space operands must share the column dimension")
    lo, hi = column_bounds(columns, rank, world_size)
    return (tensors[0], *(t[..., lo:hi] for t in tensors[1:]))


def gather_columns(shard: torch.Tensor, columns: int, group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """All-gather output shards along the last dimension into the full [..., columns] result on every rank."""
    world = dist.get_world_size(group)
    sizes = [hi - lo for lo, hi in (column_bounds(columns, r, world) for r in range(world))]
    if shard.shape[-1] != sizes[dist.get_rank(group)]:
        raise ValueError(f"shard has {shard.shape[-1]} columns, expected {sizes[dist.get_rank(group)]}")
    biggest = max(sizes)
    lead = tuple(shard.shape[:-1])
    if biggest == 0:
        return shard.new_empty((*lead, 0))
    padded = shard.new_zeros((*lead, biggest))
    padded[..., : shard.shape[-1]] = shard
    full = shard.new_empty((world * lead[0], *lead[1:], biggest))  # the ranks' shards one after another
    dist.all_gather_into_tensor(full, padded, group=group)
    full = full.view(world, *lead, biggest)
    return torch.cat([full[r][..., : sizes[r]] for r in range(world)], dim=-1)


def run_sharded(
    op: Callable[..., torch.Tensor],
    tensors: Sequence[torch.Tensor],
    *,
    gather: bool = False,
    axis: str = "auto",
    group: dist.ProcessGroup | None = None,
    **op_kwargs,
) -> torch.Tensor:
    """Apply `op` (lm2exp or lt2exp) to this rank's share of the work.  `axis="batch"` gives every rank a
    block of the batch; `axis="columns"` replicates the first operand and gives every rank a block of the K
    columns; `axis="auto"` takes the batch unless it has fewer entries than there are ranks (e.g. 4 batch
    entries on 8 GPUs).  With `gather=True` the shards are all-gathered and every rank returns the full
    result; otherwise each rank returns its own block."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    batch = tensors[0].shape[0]
    if axis not in ("auto", "batch", "columns"):
        raise ValueError(f"unknown sharding axis '{axis}'")
    if axis == "columns" or (axis == "auto" and batch < world):
        columns = tensors[-1].shape[-1]
        mine = shard_columns(tensors, rank, world)
        if mine[-1].shape[-1] > 0:
            out = op(*mine, **op_kwargs)
        else:
            out = tensors[-1].new_empty((batch, tensors[0].shape[1], 0))
        return gather_columns(out, columns, group) if gather else out
    mine = shard_batch(tensors, rank, world)
    if mine[0].shape[0] > 0:
        out = op(*mine, **op_kwargs)
    else:
        # empty shard: shape comes from the op's contract (last dim of the last operand)
        out = tensors[-1].new_empty((0, tensors[0].shape[1], tensors[-1].shape[2]))
    return gather_batch(out, batch, group) if gather else out
