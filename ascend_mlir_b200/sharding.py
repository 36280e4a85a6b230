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


class RowsumExchange:
    """The same exchange inside the reduction kernel: afirt_rowsum_exchange_* of the C-ABI library.

    Every rank reduces its column slice and stores each partial row sum straight into all ranks' mailboxes over
    NVLink as an 8-byte {sum, call number} entry; the warp that sent a row reads the other ranks' entries for it one
    row later (waiting 2 s at most) and adds them in rank order.  One launch per rank, no library collective,
    identical bits on every rank.  `connect()` gathers the mailbox
    handles over the default process group (any backend; objects, not tensors); `connect_handles()` takes them
    from elsewhere.  Every rank needs a GPU of its own."""

    ELEM_TYPES = {"f32": 0, "f16": 1, "bf16": 2}

    def __init__(self, device_id: int, rank: int, world_size: int, max_rows: int):
        import ctypes
        from .runtime._capi import EXCHANGE_HANDLE_BYTES, get_lib
        self._ct = ctypes
        self._lib = get_lib()
        self.rank, self.world_size, self.max_rows = rank, world_size, max_rows
        self._ptr = ctypes.c_void_p()
        handle = (ctypes.c_uint8 * EXCHANGE_HANDLE_BYTES)()
        err = ctypes.create_string_buffer(512)
        if self._lib.afirt_rowsum_exchange_create(device_id, rank, world_size, max_rows, ctypes.byref(self._ptr), handle,
                                                  err, len(err)):
            raise RuntimeError(err.value.decode())
        self.handle = bytes(handle)

    @property
    def pointer(self):
        """The AfirtRowsumExchange handle as a ctypes pointer (CudaRuntime.launch_device(exchange=...) takes the object)."""
        return self._ptr

    def connect_handles(self, handles) -> None:
        ct = self._ct
        blob = b"".join(handles)
        arr = (ct.c_uint8 * len(blob)).from_buffer_copy(blob)
        err = ct.create_string_buffer(512)
        if len(handles) != self.world_size:
            raise ValueError(f"{len(handles)} handles for a world of {self.world_size}")
        if self._lib.afirt_rowsum_exchange_connect(self._ptr, arr, err, len(err)):
            raise RuntimeError(err.value.decode())

    def connect(self) -> None:
        if self.world_size == 1:
            return self.connect_handles([self.handle])
        import torch.distributed as dist
        handles = [None] * self.world_size
        dist.all_gather_object(handles, self.handle)
        self.connect_handles(handles)

    def bcast_add_rowsum(self, a_ptr: int, b_ptr: int, out_ptr: int, rows: int, cols: int, b_row_stride: int,
                         elem_type: str = "f32", stream: int = 0) -> None:
        """Enqueues out[m] = sum over ranks of sum_n (a[m] + b_r[m, n]); the pointers are device addresses."""
        ct = self._ct
        err = ct.create_string_buffer(512)
        if self._lib.afirt_bcast_add_rowsum_exchange(self._ptr, self.ELEM_TYPES[elem_type], ct.c_void_p(a_ptr), ct.c_void_p(b_ptr),
                                                     ct.c_void_p(out_ptr), rows, cols, b_row_stride, ct.c_void_p(stream),
                                                     err, len(err)):
            raise RuntimeError(err.value.decode())

    def bcast_add_rowsum_batch(self, a_ptrs, b_ptrs, out_ptrs, rows: int, cols: int, b_row_stride: int,
                               elem_type: str = "f32", stream: int = 0) -> None:
        """Enqueues len(a_ptrs) independent reductions of one shape back to back with one call into the library."""
        ct = self._ct
        n = len(a_ptrs)
        arr = lambda ptrs: (ct.c_void_p * n)(*ptrs)  # noqa: E731
        err = ct.create_string_buffer(512)
        if self._lib.afirt_bcast_add_rowsum_exchange_batch(self._ptr, self.ELEM_TYPES[elem_type], n, arr(a_ptrs), arr(b_ptrs),
                                                           arr(out_ptrs), rows, cols, b_row_stride, ct.c_void_p(stream),
                                                           err, len(err)):
            raise RuntimeError(err.value.decode())

    def check(self) -> None:
        """After the stream has been synchronised: raises when a wait inside the kernel ran out."""
        err = self._ct.create_string_buffer(512)
        if self._lib.afirt_rowsum_exchange_status(self._ptr, err, len(err)):
            raise RuntimeError(err.value.decode())

    def close(self) -> None:
        if self._ptr:
            self._lib.afirt_rowsum_exchange_destroy(self._ptr)
            self._ptr = self._ct.c_void_p()


# ---- operands on other GPUs of the node: afirt_peer_* of the C-ABI library ----------------------------------------
def export_peer(device_ptr: int) -> bytes:
    """Handle (bytes) that lets another process on this node map the device memory at `device_ptr`."""
    import ctypes
    from .runtime._capi import PEER_HANDLE_BYTES, get_lib
    handle = (ctypes.c_uint8 * PEER_HANDLE_BYTES)()
    err = ctypes.create_string_buffer(512)
    if get_lib().afirt_peer_export(ctypes.c_void_p(device_ptr), handle, err, len(err)):
        raise RuntimeError(err.value.decode())
    return bytes(handle)


def import_peer(device_id: int, handle: bytes) -> int:
    """Device address, valid on `device_id` in this process, of the memory another process exported."""
    import ctypes
    from .runtime._capi import get_lib
    arr = (ctypes.c_uint8 * len(handle)).from_buffer_copy(handle)
    out = ctypes.c_void_p()
    err = ctypes.create_string_buffer(512)
    if get_lib().afirt_peer_import(device_id, arr, ctypes.byref(out), err, len(err)):
        raise RuntimeError(err.value.decode())
    return int(out.value)


def release_peer(device_ptr: int) -> None:
    import ctypes
    from .runtime._capi import get_lib
    err = ctypes.create_string_buffer(512)
    if get_lib().afirt_peer_release(ctypes.c_void_p(device_ptr), err, len(err)):
        raise RuntimeError(err.value.decode())


class ShardedTable:
    """A gather table whose rows are split over the ranks' GPUs: rank r keeps rows [r * R, (r + 1) * R) in
    `local_shard` (a contiguous CUDA tensor of R rows; the last rank's may be shorter).  After construction
    `pointers[s]` is shard s as this rank's GPU addresses it (its own shard directly, the others through CUDA IPC),
    ready for CudaRuntime.launch_device(table_shards=table.pointers, rows_per_shard=table.rows_per_shard).
    The exchange of handles uses the default process group (objects; any backend).  Keep `local_shard` alive until
    every rank has called close()."""

    def __init__(self, local_shard, device_id: int, rows_per_shard: int):
        rank, size = world()
        self.local_shard, self.device_id, self.rows_per_shard = local_shard, device_id, rows_per_shard
        mine = export_peer(local_shard.data_ptr())
        handles = [mine]
        if size > 1:
            import torch.distributed as dist
            handles = [None] * size
            dist.all_gather_object(handles, mine)
        self._imported = []
        self.pointers = []
        for r, h in enumerate(handles):
            if r == rank:
                self.pointers.append(local_shard.data_ptr())
            else:
                p = import_peer(device_id, h)
                self._imported.append(p)
                self.pointers.append(p)

    def close(self) -> None:
        for p in self._imported:
            release_peer(p)
        self._imported = []
