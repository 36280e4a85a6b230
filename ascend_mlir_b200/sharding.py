"""Row sharding across GPUs and the cross-rank bookkeeping of a sharded run.

The fused groups shard on their independent leading axis and need no data-path collective; ranks only
agree on timing (MAX over ranks) and on the total amount of work (SUM over ranks).  Works with any
torch.distributed backend (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

from typing import Optional, Tuple

from .configs import row_range  # noqa: F401  (re-exported)


def world() -> Tuple[int, int]:
    """(rank, world_size) of the default process group, (0, 1) when not initialised."""
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
    except ImportError:
        pass
    return 0, 1


def max_over_ranks(value: float, device=None) -> float:
    rank, size = world()
    if size == 1:
        return float(value)
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device=None) -> float:
    rank, size = world()
    if size == 1:
        return float(value)
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def job_throughput(work_this_rank: float, ms_this_rank: float, device=None) -> Tuple[float, float]:
    """Whole-job throughput of one sharded step: (sum of work over ranks) / (max time over ranks).

    Returns (work units per second, max milliseconds)."""
    ms = max_over_ranks(ms_this_rank, device)
    total = sum_over_ranks(work_this_rank, device)
    return total / (ms * 1e-3), ms
