"""The reduction with its exchange inside the kernel (afirt_rowsum_exchange_*), on one GPU: a world of one rank
sends its partial sums to its own mailbox, so the flag protocol, the epoch parity and both kernel variants run
without any other rank to wait for.  The two-GPU case lives in test_column_sharded_gpu.py."""
import ctypes

import numpy as np
import pytest

from ascend_mlir_b200 import descriptors
from ascend_mlir_b200.runtime._capi import get_lib
from ascend_mlir_b200.runtime.executor import CudaRuntime
from ascend_mlir_b200.sharding import RowsumExchange
from oracle import oracle

pytestmark = pytest.mark.gpu


def _ordinary(torch, rt, a, b_full, lo, hi, dtype):
    """The ordinary device entry point on the same column slice (a strided view needs a contiguous copy there)."""
    spec = descriptors.bcast_add_rowsum(dtype)
    mine = b_full[:, lo:hi].contiguous()
    out = torch.empty(a.shape[0], dtype=a.dtype, device="cuda")
    nbytes = lambda t: t.numel() * t.element_size()
    rt.launch_device(spec.binary, spec.name, [(a.data_ptr(), nbytes(a)), (mine.data_ptr(), nbytes(mine))],
                     [(out.data_ptr(), nbytes(out))], spec.pack({"M": a.shape[0], "N": hi - lo}), 0, spec.magic)
    rt.synchronize()
    return out


@pytest.mark.parametrize("rows,cols,lo,hi", [
    (2048, 4096, 0, 4096),     # whole rows: the bulk-copy staged kernel
    (2048, 8192, 4096, 8192),  # right half of wider rows (row stride > cols), staged kernel
    (300, 777, 0, 777),        # element access, few rows
    (1, 5, 1, 4),              # one row, unaligned slice
])
def test_world_of_one_matches_the_ordinary_entry_point_over_several_epochs(rows, cols, lo, hi):
    import torch
    rt = CudaRuntime()
    rt.set_device(0)
    x = RowsumExchange(0, 0, 1, max_rows=4096)
    x.connect()
    rng = np.random.default_rng(rows + cols)
    try:
        for epoch in range(4):  # both halves of the mailbox twice
            a_h = rng.uniform(-1, 1, rows).astype(np.float32)
            b_h = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
            a, b = torch.from_numpy(a_h).cuda(), torch.from_numpy(b_h).cuda()
            out = torch.full((rows,), float("nan"), device="cuda")
            x.bcast_add_rowsum(a.data_ptr(), b.data_ptr() + lo * 4, out.data_ptr(), rows, hi - lo, cols)
            torch.cuda.synchronize()
            x.check()
            want = _ordinary(torch, rt, a, b, lo, hi, "f32")
            assert torch.equal(out, want), epoch
            _, s64, abs64 = oracle.bcast_add_rowsum_f32(a_h, np.ascontiguousarray(b_h[:, lo:hi]), with_bounds=True)
            assert np.all(np.abs(out.cpu().numpy() - s64) <= 1e-5 * abs64 + 1e-30)
    finally:
        x.close()


def test_captured_calls_replay_as_a_graph():
    """The call number is kept on the device, so a captured sequence of exchange calls can be replayed: three calls
    (odd count: the replays start on alternating halves of the mailbox) captured once, replayed three times."""
    import torch
    rt = CudaRuntime()
    rt.set_device(0)
    rows, cols = 2048, 4096
    x = RowsumExchange(0, 0, 1, max_rows=rows)
    x.connect()
    try:
        g = torch.Generator(device="cuda").manual_seed(11)
        a = [torch.randn(rows, device="cuda", generator=g) for _ in range(3)]
        b = [torch.randn(rows, cols, device="cuda", generator=g) for _ in range(3)]
        out = [torch.zeros(rows, device="cuda") for _ in range(3)]
        stream = torch.cuda.Stream()
        x.bcast_add_rowsum(a[0].data_ptr(), b[0].data_ptr(), out[0].data_ptr(), rows, cols, cols, "f32", stream.cuda_stream)  # set-up outside the capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            cap = torch.cuda.current_stream().cuda_stream
            x.bcast_add_rowsum_batch([t.data_ptr() for t in a], [t.data_ptr() for t in b], [t.data_ptr() for t in out], rows, cols, cols, "f32", cap)
        want = [_ordinary(torch, rt, a[i], b[i], 0, cols, "f32") for i in range(3)]
        for replay in range(3):
            for t in out:
                t.fill_(float("nan"))
            torch.cuda.synchronize()
            with torch.cuda.stream(stream):
                graph.replay()
            stream.synchronize()
            x.check()
            for i in range(3):
                assert torch.equal(out[i], want[i]), (replay, i)
        # and an ordinary call after the replays continues the sequence
        out[0].fill_(float("nan"))
        torch.cuda.synchronize()
        x.bcast_add_rowsum(a[1].data_ptr(), b[1].data_ptr(), out[0].data_ptr(), rows, cols, cols, "f32", stream.cuda_stream)
        stream.synchronize()
        x.check()
        assert torch.equal(out[0], want[1])
    finally:
        x.close()


def test_world_of_one_bf16_rounds_once_after_the_f32_sum():
    import torch
    rt = CudaRuntime()
    rt.set_device(0)
    rows, cols = 1536, 2048
    x = RowsumExchange(0, 0, 1, max_rows=rows)
    x.connect()
    try:
        g = torch.Generator(device="cuda").manual_seed(5)
        a = torch.randn(rows, device="cuda", generator=g).to(torch.bfloat16)
        b = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
        out = torch.zeros(rows, dtype=torch.bfloat16, device="cuda")
        x.bcast_add_rowsum(a.data_ptr(), b.data_ptr(), out.data_ptr(), rows, cols, cols, "bf16")
        torch.cuda.synchronize()
        x.check()
        assert torch.equal(out, _ordinary(torch, rt, a, b, 0, cols, "bf16"))
    finally:
        x.close()


def test_compiled_row_reduction_group_through_the_exchange():
    """afirt_executor_launch_device_exchange: any row-reduction descriptor, the exchange as one more argument."""
    import torch
    from ascend_mlir_b200.runtime.executor import ExecutorError
    rt = CudaRuntime()
    rt.set_device(0)
    x = RowsumExchange(0, 0, 1, max_rows=2048)
    x.connect()
    try:
        for dtype, tdt in (("f32", torch.float32), ("f16", torch.float16)):
            spec = descriptors.bcast_add_rowsum(dtype)
            for rows, cols in ((2048, 4096), (77, 130)):
                g = torch.Generator(device="cuda").manual_seed(rows)
                a = torch.randn(rows, device="cuda", generator=g).to(tdt)
                b = torch.randn(rows, cols, device="cuda", generator=g).to(tdt)
                out = torch.zeros(rows, dtype=tdt, device="cuda")
                nb = lambda t: t.numel() * t.element_size()
                rt.launch_device(spec.binary, spec.name, [(a.data_ptr(), nb(a)), (b.data_ptr(), nb(b))], [(out.data_ptr(), nb(out))],
                                 spec.pack({"M": rows, "N": cols}), 0, spec.magic, exchange=x)
                rt.synchronize()
                x.check()
                assert torch.equal(out, _ordinary(torch, rt, a, b, 0, cols, dtype)), (dtype, rows, cols)
        # too many rows for the mailbox, and a class that has nothing to exchange
        a = torch.zeros(4096, device="cuda")
        b = torch.zeros(4096, 8, device="cuda")
        out = torch.zeros(4096, device="cuda")
        spec = descriptors.bcast_add_rowsum("f32")
        with pytest.raises(ExecutorError, match="max_rows"):
            rt.launch_device(spec.binary, spec.name, [(a.data_ptr(), 4096 * 4), (b.data_ptr(), 4096 * 32)], [(out.data_ptr(), 4096 * 4)],
                             spec.pack({"M": 4096, "N": 8}), 0, spec.magic, exchange=x)
        ew = descriptors.add_mul("f32")
        m = torch.zeros(8, 8, device="cuda")
        with pytest.raises(ExecutorError, match="only a single row-reduction group"):
            rt.launch_device(ew.binary, ew.name, [(m.data_ptr(), 256), (m.data_ptr(), 256)], [(m.data_ptr(), 256)],
                             ew.pack({"M": 8, "N": 8}), 0, ew.magic, exchange=x)
        # the refused calls did not count: the next one still works
        a = torch.ones(16, device="cuda"); b = torch.ones(16, 4, device="cuda"); out = torch.zeros(16, device="cuda")
        x.bcast_add_rowsum(a.data_ptr(), b.data_ptr(), out.data_ptr(), 16, 4, 4)
        torch.cuda.synchronize()
        x.check()
        assert torch.equal(out, torch.full((16,), 8.0, device="cuda"))
    finally:
        x.close()


def test_argument_errors_leave_the_exchange_usable():
    import torch
    lib = get_lib()
    x = RowsumExchange(0, 0, 1, max_rows=64)
    a = torch.ones(64, device="cuda")
    b = torch.ones(64, 8, device="cuda")
    out = torch.zeros(64, device="cuda")
    with pytest.raises(RuntimeError, match="not connected"):
        x.bcast_add_rowsum(a.data_ptr(), b.data_ptr(), out.data_ptr(), 64, 8, 8)
    with pytest.raises(RuntimeError, match="not this exchange's own"):
        x.connect_handles([bytes(x.handle[:72]) + b"\x01" + bytes(x.handle[73:])])  # another owner's address
    x.connect()
    with pytest.raises(RuntimeError, match="already connected"):
        x.connect()
    with pytest.raises(RuntimeError, match="max_rows"):
        x.bcast_add_rowsum(a.data_ptr(), b.data_ptr(), out.data_ptr(), 65, 8, 8)
    with pytest.raises(RuntimeError, match="b_row_stride"):
        x.bcast_add_rowsum(a.data_ptr(), b.data_ptr(), out.data_ptr(), 64, 8, 4)
    x.bcast_add_rowsum(a.data_ptr(), b.data_ptr(), out.data_ptr(), 64, 8, 8)
    torch.cuda.synchronize()
    x.check()
    assert torch.equal(out, torch.full((64,), 16.0, device="cuda"))
    x.close()
    err = ctypes.create_string_buffer(64)
    assert lib.afirt_rowsum_exchange_status(None, err, len(err)) == 1 and err.value


def test_batch_call_enqueues_independent_reductions_back_to_back():
    """afirt_bcast_add_rowsum_exchange_batch: five reductions (five operand sets, five outputs) by one call; each gets
    its own call number, so the mailbox halves alternate exactly as with five single calls."""
    import torch
    rt = CudaRuntime()
    rt.set_device(0)
    rows, cols = 2048, 4096
    x = RowsumExchange(0, 0, 1, max_rows=rows)
    x.connect()
    try:
        g = torch.Generator(device="cuda").manual_seed(9)
        sets = [(torch.rand(rows, device="cuda", generator=g) - 0.5, torch.rand(rows, cols, device="cuda", generator=g) - 0.5)
                for _ in range(5)]
        outs = [torch.full((rows,), float("nan"), device="cuda") for _ in sets]
        x.bcast_add_rowsum_batch([a.data_ptr() for a, _ in sets], [b.data_ptr() for _, b in sets], [o.data_ptr() for o in outs],
                                 rows, cols, cols)
        torch.cuda.synchronize()
        x.check()
        for (a, b), out in zip(sets, outs):
            assert torch.equal(out, _ordinary(torch, rt, a, b, 0, cols, "f32"))
        x.bcast_add_rowsum_batch([], [], [], rows, cols, cols)  # an empty batch is a no-op
    finally:
        x.close()
