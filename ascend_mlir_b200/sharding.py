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


# ---- the one exchange step of the path: a reduction whose axis is sharded ---------------------------------------
def col_range(total: int, rank: int, world_size: int, quantum: int = 1) -> Tuple[int, int]:
    """Contiguous, balanced partition of `total` columns in units of `quantum` (e.g. 4 for 16-byte f32 vectors)."""
    units = (total + quantum - 1) // quantum
    lo, hi = row_range(units, rank, world_size)
    return min(total, lo * quantum), min(total, hi * quantum)


def allreduce_partial_rowsums(partial):
    """Sums per-rank partial row sums in place across the default process group and returns the tensor.

    Row sharding (the default for every group) needs no collective.  When the *reduced* axis is sharded instead
    (each rank holds a column slice of x), every rank reduces its slice with the row-reduction kernel in f32 and the
    partial sums are added here: one all-reduce of rows x 4 bytes (32 KiB for 8192 rows), NCCL over NVLink on GPUs,
    gloo on CPU.  The broadcast operand b[m] must be added on one rank only (or scaled by the slice widths), which
    is why the helper takes finished partial sums and not the operands."""
    rank, size = world()
    if size == 1:
        return partial
    import torch.distributed as dist
    dist.all_reduce(partial, op=dist.ReduceOp.SUM)
    return partial
