"""One process, two GPUs: an executor per device.  Function attributes (the opt-in to more than 48 KB of dynamic
shared memory) and loaded modules belong to a device, so what was set up by the first executor on device 0 must be
set up again for the second one on device 1: the matmul (tcgen05 kernel, 200 KB of shared memory), the staged row
reduction (128 KB) and a generated kernel (a module loaded per executor)."""
import numpy as np
import pytest

from ascend_mlir_b200 import configs
from ascend_mlir_b200.runtime.executor import CudaRuntime
from oracle import oracle

pytestmark = pytest.mark.gpu


def _two_gpus():
    import torch
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2


@pytest.mark.skipif(not _two_gpus(), reason="needs two GPUs")
def test_same_descriptors_on_device_0_then_device_1():
    import torch
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")  # this thread now has device 0 current, as a framework-hosted caller would
    runtimes = []
    for device in (0, 1):
        rt = CudaRuntime()
        rt.set_device(device)
        runtimes.append(rt)
    mm = configs.matmul_add_leakyrelu(512, 768, 320, seed=3)
    want_mm = oracle.bf16_to_f32(oracle.matmul_bias_leakyrelu_bf16(*mm.inputs, 0.01))
    red = configs.broadcast_add_reduce(1500, 8192, seed=4)   # long rows, enough of them: the staged kernel
    _, s64, abs64 = oracle.bcast_add_rowsum_f32(red.inputs[0], red.inputs[1], with_bounds=True)
    ew = configs.chain_sub_div_min(300, 520, seed=5)          # a generated kernel
    for rt in runtimes:
        out = mm.new_output()
        rt.run(mm.spec.binary, mm.spec.name, mm.inputs, [out], mm.tiling(), magic=mm.spec.magic)
        got = oracle.bf16_to_f32(out)
        assert np.all(np.abs(got - want_mm) <= 1e-2 * np.abs(want_mm) + 1e-3)
        out = red.new_output()
        rt.run(red.spec.binary, red.spec.name, red.inputs, [out], red.tiling())
        assert np.all(np.abs(out - s64) <= 1e-5 * abs64)
        out = ew.new_output()
        rt.run(ew.spec.binary, ew.spec.name, ew.inputs, [out], ew.tiling())
        assert rt.last_launch_generated
        assert np.array_equal(out, ew.expected())
        # the library made its own device current for the calls and put the caller's back
        assert torch.cuda.current_device() == 0
