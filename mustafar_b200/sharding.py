"""Batch / kv-head sharding of the sparse cache across ranks.

Every (sequence, kv head) is an independent unit of the hot path (compression, append, decode
attention), so ranks own disjoint contiguous ranges of units and never exchange cache data; the
only collective a benchmark or a server needs is the reduction of its own timings or results.
"""
from __future__ import annotations


def shard_range(n_units: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous [begin, end) of `n_units` owned by `rank`; sizes differ by at most one."""
    if not (0 <= rank < world) or n_units < 0:
        raise ValueError("bad rank / world / n_units")
    base, rem = divmod(n_units, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def max_over_ranks(value: float, dist=None, device=None) -> float:
    """Device timings are reported as the maximum over ranks (the slowest rank ends the step)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])
