"""Batch-dimension sharding of lm2exp / lt2exp across the GPUs of one node.

Every batch entry r of both ops is independent (the reference's kernels only use the batch index to offset
pointers, triturus/lm2exp.py:94,122-123 and triturus/lt2exp.py:264,301-303), so the multi-GPU path is one
process per GPU, each owning a contiguous block of r, with no collective on the data path.  The only
communication offered is an optional all-gather of the output shards (`gather_batch`), which callers time
and report separately.  Works with the NCCL backend on GPUs and the gloo backend on CPU tensors.
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


def run_sharded(
    op: Callable[..., torch.Tensor],
    tensors: Sequence[torch.Tensor],
    *,
    gather: bool = False,
    group: dist.ProcessGroup | None = None,
    **op_kwargs,
) -> torch.Tensor:
    """Apply `op` (lm2exp or lt2exp) to this rank's block of the batch.  With `gather=True` the shards are
    all-gathered and every rank returns the full result; otherwise each rank returns its own block."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    batch = tensors[0].shape[0]
    mine = shard_batch(tensors, rank, world)
    if mine[0].shape[0] > 0:
        out = op(*mine, **op_kwargs)
    else:
        # empty shard: shape comes from the op's contract (last dim of the last operand)
        out = tensors[-1].new_empty((0, tensors[0].shape[1], tensors[-1].shape[2]))
    return gather_batch(out, batch, group) if gather else out
