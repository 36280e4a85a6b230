"""Kernel executor (counterpart of the reference's python/runtime/executor.py) over the afirt_* C-ABI.

Host path: `CudaRuntime.run` takes numpy arrays, as the reference's AscendRuntime.run does.
Device path: `CudaRuntime.launch_device` takes raw device pointers + byte counts and a CUDA stream
handle, for callers whose tensors already live in GPU memory.
"""
import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ._capi import get_lib
from .utils import SM_100A, ExecutorError

MAGIC_ELF_AIVEC = 0x41415246
MAGIC_ELF_AICUBE = 0x41494343

_u8p = ctypes.POINTER(ctypes.c_uint8)


def _u8(data: Optional[bytes]):
    if not data:
        return ctypes.cast(ctypes.c_void_p(0), _u8p), 0, None
    arr = (ctypes.c_uint8 * len(data)).from_buffer_copy(data)
    return ctypes.cast(arr, _u8p), len(data), arr


class CudaRuntime:
    MAGIC_ELF_AIVEC = MAGIC_ELF_AIVEC
    MAGIC_ELF_AICUBE = MAGIC_ELF_AICUBE

    def __init__(self, ascend_root=None, soc_version: str = SM_100A, simulation_mode: bool = False):
        self.soc_version = soc_version
        self._initialized = False
        lib = get_lib()
        handle = lib.afirt_executor_create()
        if not handle:
            raise ExecutorError("Failed to create executor instance")
        self._handle = handle
        self._keep = {}

    def __del__(self):
        if getattr(self, "_handle", None):
            try:
                get_lib().afirt_executor_destroy(ctypes.c_void_p(self._handle))
            except Exception:
                pass
            self._handle = None

    def set_device(self, device_id: int = 0):
        err = ctypes.create_string_buffer(1024)
        ret = get_lib().afirt_executor_initialize(ctypes.c_void_p(self._handle), device_id, err, len(err))
        if ret != 0:
            raise ExecutorError(err.value.decode(errors="replace"))
        self._initialized = True

    # ---- host tensors ------------------------------------------------------------------------
    def run(self, binary_data: bytes, function_name: str, inputs: List[np.ndarray], outputs: List[np.ndarray],
            tiling_data: Optional[bytes] = None, block_dim: int = 1, magic: int = MAGIC_ELF_AIVEC) -> List[np.ndarray]:
        in_bufs = [np.ascontiguousarray(x) for x in inputs]
        out_bufs = [x if x.flags["C_CONTIGUOUS"] and x.flags["WRITEABLE"] else np.ascontiguousarray(x) for x in outputs]
        self.run_raw(binary_data, function_name,
                     [(x.ctypes.data, x.nbytes) for x in in_bufs], [(x.ctypes.data, x.nbytes) for x in out_bufs],
                     tiling_data, block_dim, magic)
        for dst, src in zip(outputs, out_bufs):
            if dst is not src:
                dst[...] = src
        return outputs

    def run_raw(self, binary_data: bytes, function_name: str, inputs: Sequence[Tuple[int, int]],
                outputs: Sequence[Tuple[int, int]], tiling_data: Optional[bytes] = None, block_dim: int = 0,
                magic: int = MAGIC_ELF_AIVEC) -> None:
        """Host path on raw (address, nbytes) pairs, e.g. pinned torch tensors."""
        lib = get_lib()
        bin_ptr, bin_len, _k1 = self._binary(binary_data)
        til_ptr, til_len, _k2 = _u8(tiling_data)
        in_ptrs = (ctypes.c_void_p * max(1, len(inputs)))(*[p for p, _ in inputs])
        in_bytes = (ctypes.c_size_t * max(1, len(inputs)))(*[n for _, n in inputs])
        out_ptrs = (ctypes.c_void_p * max(1, len(outputs)))(*[p for p, _ in outputs])
        out_bytes = (ctypes.c_size_t * max(1, len(outputs)))(*[n for _, n in outputs])
        err = ctypes.create_string_buffer(1024)
        ret = lib.afirt_executor_run(ctypes.c_void_p(self._handle), bin_ptr, bin_len, function_name.encode(),
                                     len(inputs), in_ptrs, in_bytes, len(outputs), out_ptrs, out_bytes, til_ptr, til_len,
                                     block_dim, magic, err, len(err))
        if ret != 0:
            raise ExecutorError(err.value.decode(errors="replace"))

    def run_file(self, binary_path: str, function_name: str, inputs: List[np.ndarray], outputs: List[np.ndarray],
                 tiling_data: Optional[bytes] = None, block_dim: int = 1, magic: int = MAGIC_ELF_AIVEC):
        lib = get_lib()
        in_bufs = [np.ascontiguousarray(x) for x in inputs]
        til_ptr, til_len, _k = _u8(tiling_data)
        in_ptrs = (ctypes.c_void_p * max(1, len(in_bufs)))(*[x.ctypes.data for x in in_bufs])
        in_bytes = (ctypes.c_size_t * max(1, len(in_bufs)))(*[x.nbytes for x in in_bufs])
        out_ptrs = (ctypes.c_void_p * len(outputs))(*[x.ctypes.data for x in outputs])
        out_bytes = (ctypes.c_size_t * len(outputs))(*[x.nbytes for x in outputs])
        err = ctypes.create_string_buffer(1024)
        ret = lib.afirt_executor_run_file(ctypes.c_void_p(self._handle), str(binary_path).encode(), function_name.encode(),
                                          len(in_bufs), in_ptrs, in_bytes, len(outputs), out_ptrs, out_bytes, til_ptr,
                                          til_len, block_dim, magic, err, len(err))
        if ret != 0:
            raise ExecutorError(err.value.decode(errors="replace"))
        return outputs

    # ---- device tensors ----------------------------------------------------------------------
    def launch_device(self, binary_data: bytes, function_name: str, inputs: Sequence[Tuple[int, int]],
                      outputs: Sequence[Tuple[int, int]], tiling_data: Optional[bytes] = None, block_dim: int = 0,
                      magic: int = MAGIC_ELF_AIVEC, workspace: Tuple[int, int] = (0, 0), stream: int = 0,
                      exchange=None, table_shards=None, rows_per_shard: int = 0) -> None:
        """Enqueue on `stream` (a cudaStream_t as int); inputs/outputs are (device address, nbytes).

        `exchange` (a connected sharding.RowsumExchange) makes a row-reduction group exchange its partial sums with
        the other ranks inside the kernel: the arguments are this rank's column slice, the output the full sums.
        `table_shards` (device addresses, other GPUs' memory included) with `rows_per_shard` gives the table of a
        row-gather group as row shards; the table's own entry in `inputs` then only carries the whole table's size."""
        lib = get_lib()
        bin_ptr, bin_len, _k1 = self._binary(binary_data)
        til_ptr, til_len, _k2 = _u8(tiling_data)
        in_ptrs = (ctypes.c_void_p * max(1, len(inputs)))(*[p for p, _ in inputs])
        in_bytes = (ctypes.c_size_t * max(1, len(inputs)))(*[n for _, n in inputs])
        out_ptrs = (ctypes.c_void_p * max(1, len(outputs)))(*[p for p, _ in outputs])
        out_bytes = (ctypes.c_size_t * max(1, len(outputs)))(*[n for _, n in outputs])
        err = ctypes.create_string_buffer(1024)
        head = (ctypes.c_void_p(self._handle), bin_ptr, bin_len, function_name.encode(), len(inputs), in_ptrs, in_bytes,
                len(outputs), out_ptrs, out_bytes, til_ptr, til_len, block_dim, magic, ctypes.c_void_p(workspace[0]),
                workspace[1], ctypes.c_void_p(stream))
        if table_shards is not None:
            shards = (ctypes.c_void_p * len(table_shards))(*table_shards)
            ret = lib.afirt_executor_launch_device_sharded_table(*head, len(table_shards), shards, rows_per_shard, err, len(err))
        elif exchange is None:
            ret = lib.afirt_executor_launch_device(*head, err, len(err))
        else:
            ret = lib.afirt_executor_launch_device_exchange(*head, exchange.pointer, err, len(err))
        if ret != 0:
            raise ExecutorError(err.value.decode(errors="replace"))

    def synchronize(self, stream: int = 0) -> None:
        err = ctypes.create_string_buffer(1024)
        if get_lib().afirt_executor_synchronize(ctypes.c_void_p(self._handle), ctypes.c_void_p(stream), err, len(err)) != 0:
            raise ExecutorError(err.value.decode(errors="replace"))

    def workspace_bytes(self, binary_data: bytes, tiling_data: Optional[bytes]) -> int:
        bin_ptr, bin_len, _k1 = self._binary(binary_data)
        til_ptr, til_len, _k2 = _u8(tiling_data)
        out = ctypes.c_size_t(0)
        err = ctypes.create_string_buffer(1024)
        if get_lib().afirt_executor_workspace_bytes(ctypes.c_void_p(self._handle), bin_ptr, bin_len, til_ptr, til_len,
                                                    ctypes.byref(out), err, len(err)) != 0:
            raise ExecutorError(err.value.decode(errors="replace"))
        return int(out.value)

    @property
    def last_launch_count(self) -> int:
        return int(get_lib().afirt_executor_last_launch_count(ctypes.c_void_p(self._handle)))

    @property
    def last_launch_generated(self) -> bool:
        """True when the last launch ran the group's generated kernel, False when it ran a prebuilt library kernel."""
        return bool(get_lib().afirt_executor_last_launch_generated(ctypes.c_void_p(self._handle)))

    @property
    def total_launch_count(self) -> int:
        return int(get_lib().afirt_executor_total_launch_count(ctypes.c_void_p(self._handle)))

    def _binary(self, binary_data: bytes):
        # ctypes copies of the (small) binary are cached so repeated launches do not re-copy
        key = id(binary_data)
        hit = self._keep.get(key)
        if hit is None or hit[3] is not binary_data:
            ptr, n, arr = _u8(binary_data)
            hit = (ptr, n, arr, binary_data)
            if len(self._keep) > 64:
                self._keep.clear()
            self._keep[key] = hit
        return hit[0], hit[1], hit[2]


AscendRuntime = CudaRuntime  # name used by callers of the reference package


class KernelExecutor:
    def __init__(self, ascend_root=None, soc_version: str = SM_100A, device_id: int = 0, simulation_mode: bool = False):
        self.runtime = CudaRuntime(ascend_root, soc_version, simulation_mode)
        self.device_id = device_id
        self._initialized = False

    def initialize(self):
        self.runtime.set_device(self.device_id)
        self._initialized = True

    def execute(self, binary_data: bytes, function_name: str, inputs: List[np.ndarray], outputs: List[np.ndarray],
                tiling_data: Optional[bytes] = None, block_dim: int = 1, magic: int = MAGIC_ELF_AIVEC) -> List[np.ndarray]:
        if not self._initialized:
            self.initialize()
        return self.runtime.run(binary_data, function_name, inputs, outputs, tiling_data, block_dim, magic)


def execute_kernel(binary_data: bytes, function_name: str, inputs: List[np.ndarray],
                   output_shapes: List[Tuple[int, ...]], tiling_data: Optional[bytes] = None, ascend_root=None,
                   soc_version: str = SM_100A, device_id: int = 0, dtype=np.float32,
                   simulation_mode: bool = False, block_dim: int = 0) -> List[np.ndarray]:
    outputs = [np.zeros(shape, dtype=dtype) for shape in output_shapes]
    executor = KernelExecutor(ascend_root, soc_version, device_id, simulation_mode)
    return executor.execute(binary_data, function_name, inputs, outputs, tiling_data, block_dim=block_dim)
