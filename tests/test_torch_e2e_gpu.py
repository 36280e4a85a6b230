"""torch_e2e on the GPU: the decorated tests of the reference's examples/torch_e2e/test_elementwise.py (same
models and shape patterns), plus a matmul model and a direct comparison of the kernel output with eager PyTorch.
Each decorated test passes when the autotuner has compiled the group, run every tiling candidate and found each
within tolerance of the eager result."""
import json
import warnings

import numpy as np
import pytest
import torch

from ascend_mlir_b200 import build as lib_build
from ascend_mlir_b200.torch_e2e import TensorSpec, compile_model, run_autotuner, torch_e2e_test

pytestmark = pytest.mark.gpu
warnings.filterwarnings("ignore", category=FutureWarning)


@pytest.fixture(scope="module", autouse=True)
def built(tmp_path_factory):
    lib_build.build()
    mp = pytest.MonkeyPatch()
    mp.setenv("AFIR_TORCH_E2E_OUTPUT", str(tmp_path_factory.mktemp("torch_e2e")))
    yield
    mp.undo()


@torch_e2e_test
def test_add_mul():
    class Model(torch.nn.Module):
        def forward(self, a, b, c):
            return (a + b) * c

    return Model(), [TensorSpec(("M", "N"))] * 3


@torch_e2e_test
def test_add_reduce():
    class Model(torch.nn.Module):
        def forward(self, a, b):
            return (a + b).sum(dim=1)

    return Model(), [TensorSpec(("M", "N"))] * 2


@torch_e2e_test(verify_shapes={"M": 128, "N": 16})
def test_broadcast_add_reduce():
    class Model(torch.nn.Module):
        def forward(self, a, b):
            return (a.unsqueeze(1) + b).sum(dim=1)

    return Model(), [TensorSpec(("M",)), TensorSpec(("M", "N"))]


@torch_e2e_test(verify_shapes={"M": 320}, atol=2e-2, rtol=2e-2)
def test_addmm_leaky_relu():
    class Model(torch.nn.Module):
        def forward(self, x, w, bias):
            return torch.nn.functional.leaky_relu(torch.addmm(bias, x, w), 0.01)

    return Model(), [TensorSpec(("M", 256), torch.bfloat16), TensorSpec((256, 128), torch.bfloat16),
                     TensorSpec((128,), torch.bfloat16)]


@torch_e2e_test(verify_shapes={"M": 200}, atol=2e-2, rtol=2e-2)
def test_linear_module_with_its_own_weights():
    """torch.nn.Linear keeps its weight as [N, K]: the parameters become trailing kernel arguments and the matmul
    reads the weight K-major, no transposed copy."""
    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(3)
            self.fc = torch.nn.Linear(256, 384).to(torch.bfloat16)

        def forward(self, x):
            return torch.nn.functional.leaky_relu(self.fc(x), 0.01)

    return Model(), [TensorSpec(("M", 256), torch.bfloat16)]


@torch_e2e_test(atol=0.0, rtol=0.0)
def test_attention_heads_permutation():
    class Model(torch.nn.Module):
        def forward(self, x):
            return x.permute(0, 2, 1, 3).contiguous()

    return Model(), [TensorSpec((4, 24, 6, 64), torch.float16)]


@torch_e2e_test(verify_shapes={"M": 264, "N": 520}, atol=0.0, rtol=0.0)
def test_transposed_operand_clamp_abs():
    class Model(torch.nn.Module):
        def forward(self, a, b):
            return torch.clamp((a.t() + b).abs(), 0.1, 2.0)

    return Model(), [TensorSpec(("M", "N"), torch.float32), TensorSpec(("N", "M"), torch.float32)]


def test_kernel_output_matches_eager_bit_for_bit_on_f32_elementwise(tmp_path):
    """f32 elementwise chains have no rounding freedom: run the compiled group through the runtime and compare."""
    from ascend_mlir_b200.runtime import CudaRuntime, TilingSchema, compile_kernel

    class Model(torch.nn.Module):
        def forward(self, x, row):
            return torch.relu(x * 0.5 - row) / 2.0

    specs = [TensorSpec(("M", "N"), torch.float32), TensorSpec(("N",), torch.float32)]
    built = compile_model(Model(), specs, tmp_path / "ew", verify_shapes={"M": 257, "N": 1000})
    best = run_autotuner(tmp_path / "ew", 2, built["shape"], atol=0.0, rtol=0.0)
    assert best["best"]["max_abs_diff"] == 0.0

    binary = compile_kernel(str(built["kernel"]), str(tmp_path / "ew" / "art"), "forward").read_bytes()
    shape = dict(kv.split("=") for kv in built["shape"].split(","))
    fields = json.loads(built["space"].read_text())["tiling_params"]
    params = {p["name"]: int(shape[p["shape_key"]]) if p.get("fixed") else int(best["config"][p["name"]]) for p in fields}
    x, row = (t.numpy() for t in built["inputs"])
    out = np.empty((257, 1000), np.float32)
    rt = CudaRuntime()
    rt.set_device(0)
    rt.run(binary, "forward", [x, row], [out], TilingSchema.from_json(built["space"]).pack(**params), 0)
    assert np.array_equal(out, built["expected"].numpy())
