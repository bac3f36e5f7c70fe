"""Multi-GPU sharding of the neighbourhood-attention path.

Every (batch element, kv-head group) is independent: no halo, no exchange, so
ranks never communicate on the data path.  This module only decides which units
a rank owns and reduces scalars (timings, checksums) across ranks for reporting.
"""
from __future__ import annotations

from typing import List, Sequence


def assign_units(costs: Sequence[float], world_size: int) -> List[List[int]]:
    """Greedy longest-first assignment of work units (e.g. one per batch element,
    cost = its valid length) to ranks; returns the unit indices per rank.  With
    equal costs this is a round-robin split; the result is deterministic."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(costs)), key=lambda i: (-float(costs[i]), i))
    loads = [0.0] * world_size
    owned: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        owned[r].append(i)
        loads[r] += float(costs[i])
    return [sorted(u) for u in owned]


def batch_slice(batch: int, rank: int, world_size: int) -> slice:
    """Contiguous batch-major split (remainder spread over the first ranks)."""
    base, rem = divmod(batch, world_size)
    start = rank * base + min(rank, rem)
    return slice(start, start + base + (1 if rank < rem else 0))


def reduce_max(values: Sequence[float], device=None) -> List[float]:
    """Max over ranks of each value (identity when torch.distributed is not initialised)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def reduce_sum(values: Sequence[float], device=None) -> List[float]:
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.tolist()
