"""The allocation-free reduction entry point, afirt_bcast_add_rowsum_no_alloc.

Who needs it: callers that are not allowed to allocate GPU memory at call time -- serving or
real-time loops whose memory was budgeted and frozen at start-up, processes whose device memory is
already fully committed, plugins hosted by a framework that owns the device allocator.  Its scratch (the per-slice partial sums of the
column-sliced row reduction) is a fixed array inside the library, not an allocated workspace.

The test drives it through the C-ABI twice in a row with different data and compares each result with
the ordinary device entry point (afirt_executor_launch_device, workspace supplied by the caller) run
with the same column split: same kernels, same slice order, so the outputs must be identical, and
both must sit inside the reduction bound the other tests use.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest

from ascend_mlir_b200 import configs
from ascend_mlir_b200.runtime._capi import get_lib
from ascend_mlir_b200.runtime.executor import CudaRuntime
from oracle import oracle

pytestmark = pytest.mark.gpu


def _no_alloc(lib, torch, a, b, out, rows, cols, split, stream=0, elem_type=0):
    err = ctypes.create_string_buffer(256)
    rc = lib.afirt_bcast_add_rowsum_no_alloc(0, elem_type, a.data_ptr(), b.data_ptr(), out.data_ptr(), rows, cols, split,
                                            ctypes.c_void_p(stream), err, len(err))
    return rc, err.value.decode()


def test_no_alloc_matches_workspace_entry_point_twice_in_a_row():
    import torch
    lib = get_lib()
    dev = torch.device("cuda", 0)
    rt = CudaRuntime()
    rt.set_device(0)
    rows, cols, split = 48, 50000, 7
    for seed in (31, 32):  # second call reuses the scratch the first one left behind
        w = configs.broadcast_add_reduce(rows, cols, seed=seed)
        a = torch.from_numpy(w.inputs[0]).to(dev)
        b = torch.from_numpy(w.inputs[1]).to(dev)
        out_new = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
        out_old = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
        torch.cuda.synchronize()

        free_before, _ = torch.cuda.mem_get_info(dev)
        rc, msg = _no_alloc(lib, torch, a, b, out_new, rows, cols, split)
        assert rc == 0, msg
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(dev)
        if seed == 32:  # the first call may load the kernel image; the second must not move the free-memory mark
            assert free_before == free_after

        tiling = w.tiling(SPLIT_N=split)
        ws = torch.zeros(rt.workspace_bytes(w.spec.binary, tiling), dtype=torch.uint8, device=dev)
        rt.launch_device(w.spec.binary, w.spec.name,
                         [(a.data_ptr(), a.numel() * 4), (b.data_ptr(), b.numel() * 4)], [(out_old.data_ptr(), rows * 4)],
                         tiling, 0, w.spec.magic, (ws.data_ptr(), ws.numel()), 0)
        rt.synchronize(0)
        assert rt.last_launch_count == 2

        got, ref = out_new.cpu().numpy(), out_old.cpu().numpy()
        assert np.array_equal(got, ref)
        _, s64, abs64 = oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1], with_bounds=True)
        assert np.all(np.abs(got - s64) <= 1e-5 * abs64)


def test_no_alloc_without_column_slices_takes_the_staged_kernel():
    """split_cols = 1 uses no scratch at all; from 148 x 8 rows of 16 KB up the launch is the bulk-copy staged kernel
    with its 128 KB of dynamic shared memory, which must not allocate either."""
    import torch
    lib = get_lib()
    dev = torch.device("cuda", 0)
    rt = CudaRuntime()
    rt.set_device(0)
    rows, cols = 1200, 8192
    for seed in (41, 42):
        w = configs.broadcast_add_reduce(rows, cols, seed=seed)
        a = torch.from_numpy(w.inputs[0]).to(dev)
        b = torch.from_numpy(w.inputs[1]).to(dev)
        out_new = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
        out_old = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(dev)
        rc, msg = _no_alloc(lib, torch, a, b, out_new, rows, cols, 1)
        assert rc == 0, msg
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(dev)
        if seed == 42:
            assert free_before == free_after
        tiling = w.tiling(SPLIT_N=1)
        ws = torch.zeros(rt.workspace_bytes(w.spec.binary, tiling), dtype=torch.uint8, device=dev)
        rt.launch_device(w.spec.binary, w.spec.name,
                         [(a.data_ptr(), a.numel() * 4), (b.data_ptr(), b.numel() * 4)], [(out_old.data_ptr(), rows * 4)],
                         tiling, 0, w.spec.magic, (ws.data_ptr(), ws.numel()), 0)
        rt.synchronize(0)
        assert rt.last_launch_count == 1
        got = out_new.cpu().numpy()
        assert np.array_equal(got, out_old.cpu().numpy())
        _, s64, abs64 = oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1], with_bounds=True)
        assert np.all(np.abs(got - s64) <= 1e-5 * abs64)


def test_no_alloc_bf16_column_slices():
    """16-bit inputs: summed in f32, the result rounded once to bf16 (two calls in a row on the shared scratch)."""
    import torch
    lib = get_lib()
    dev = torch.device("cuda", 0)
    rows, cols, split = 64, 32768, 5
    for seed in (51, 52):
        g = torch.Generator().manual_seed(seed)
        a = (torch.rand(rows, generator=g) * 2 - 1).to(torch.bfloat16)
        b = (torch.rand(rows, cols, generator=g) * 2 - 1).to(torch.bfloat16)
        out = torch.full((rows,), float("nan"), dtype=torch.bfloat16, device=dev)
        a_dev, b_dev = a.to(dev), b.to(dev)  # kept alive until the synchronize below
        rc, msg = _no_alloc(lib, torch, a_dev, b_dev, out, rows, cols, split, elem_type=2)
        assert rc == 0, msg
        torch.cuda.synchronize()
        # per element: bf16(a + b) (one rounding), then an f64 sum as the exact reference of the f32 accumulation
        terms = (a.float()[:, None] + b.float()).to(torch.bfloat16).double()
        want = terms.sum(dim=1)
        bound = 1e-5 * terms.abs().sum(dim=1) + want.abs() * 2.0 ** -8  # accumulation bound + one bf16 rounding
        assert torch.all((out.cpu().double() - want).abs() <= bound)
    assert torch.cuda.current_device() == 0  # the entry point puts the caller's device back


def test_no_alloc_refuses_sizes_beyond_the_built_in_scratch():
    import torch
    lib = get_lib()
    dev = torch.device("cuda", 0)
    x = torch.zeros(16, dtype=torch.float32, device=dev)
    rc, msg = _no_alloc(lib, torch, x, x, x, 262144, 8, 2)
    assert rc == 1 and "exceeds the built-in scratch of 262144" in msg
    rc, msg = _no_alloc(lib, torch, x, x, x, 4, 4, 0)
    assert rc == 1 and "split_cols" in msg
    # a product that wraps around 64 bits must be refused, not pass as a small number
    rc, msg = _no_alloc(lib, torch, x, x, x, 1 << 62, 8, 4)
    assert rc == 1 and "exceeds the built-in scratch" in msg
    rc, msg = _no_alloc(lib, torch, x, x, x, 4, 1 << 41, 1)
    assert rc == 1 and "cols" in msg
