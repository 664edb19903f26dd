"""Head sharding across GPUs.

Every (batch, head) slice of the operator is an independent problem (grid
axis 1 of the reference kernels, fhog/triton_bwdbwd.py:77, :360), so N GPUs
split the folded BH axis into contiguous shards and never exchange data on
the hot path.  The only communication is the barrier and max-reduction a
benchmark or a caller needs to time the slowest rank.
"""
from __future__ import annotations

from typing import Tuple

import torch


def head_shard(total_heads: int, world_size: int, rank: int) -> Tuple[int, int]:
    """(first head, number of heads) of `rank`: contiguous, sizes differ by at most one."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} of {world_size}")
    if total_heads < 0:
        raise ValueError("total_heads must be non-negative")
    base, extra = divmod(total_heads, world_size)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def max_over_ranks(value: float, device=None, group=None) -> float:
    """Largest `value` over all ranks of the default (or given) process group; identity without one."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def sharded_call(fn, tensors, total_heads: int, world_size: int, rank: int):
    """Runs `fn` on this rank's slice of every (BH, ...) tensor in `tensors`; returns (start, count, result)."""
    start, count = head_shard(total_heads, world_size, rank)
    sl = slice(start, start + count)
    return start, count, fn(*[t[sl] for t in tensors])
