"""torch_e2e on the CPU: torch.export -> linalg text -> afir-opt -> afir-translate gives the launch descriptor
and tiling space expected for each model, the eager reference is written as .npy, and unsupported models are
refused at conversion time.  The kernels themselves run in tests/test_torch_e2e_gpu.py."""
import json
import warnings

import numpy as np
import pytest
import torch

from ascend_mlir_b200 import build as lib_build
from ascend_mlir_b200.torch_e2e import TensorSpec, UnsupportedTorchOp, compile_model, torch_to_linalg
from ascend_mlir_b200.torch_e2e.pipeline import build_shape_string

warnings.filterwarnings("ignore", category=FutureWarning)


@pytest.fixture(scope="module", autouse=True)
def built():
    lib_build.build()


class AddMul(torch.nn.Module):
    def forward(self, a, b, c):
        return (a + b) * c


class AddReduce(torch.nn.Module):
    def forward(self, a, b):
        return (a + b).sum(dim=1)


class BroadcastAddReduce(torch.nn.Module):
    def forward(self, a, b):
        return (a.unsqueeze(1) + b).sum(dim=1)


class LinearLeaky(torch.nn.Module):
    def forward(self, x, w, bias):
        return torch.nn.functional.leaky_relu(torch.addmm(bias, x, w), 0.01)


def descriptor(built):
    return json.loads(built["kernel"].read_text())


def test_tensor_spec_patterns():
    spec = TensorSpec(("M", 32, None), torch.float32)
    assert spec.make_sample({"M": 5}).shape == (5, 32, 64) and spec.make_sample().shape == (64, 32, 64)
    pool = {}
    d0, d1 = spec.dynamic_dims(pool), TensorSpec(("M",)).dynamic_dims(pool)
    assert set(d0) == {0, 2} and d0[0] is d1[0], "equal names share one symbol; static dims are left out"
    assert TensorSpec((4, 4)).dynamic_dims() == {} and TensorSpec((4,)).dtype == torch.float16


def test_add_mul_becomes_one_elementwise_group(tmp_path):
    built = compile_model(AddMul(), [TensorSpec(("M", "N"))] * 3, tmp_path / "add_mul")
    d = descriptor(built)
    assert d["kernel_class"] == "elementwise" and d["dtype"] == "f16" and d["num_inputs"] == 3
    assert [o["op"] for o in d["body"]] == ["addf", "mulf"]
    text = (tmp_path / "add_mul" / "step0_linalg.mlir").read_text()
    assert text.count("linalg.generic") == 2 and "tensor<?x?xf16>" in text
    assert built["shape"] == ",".join(f"arg{a}_dim{d}=64" for a in range(3) for d in range(2))
    for i in range(3):
        assert np.load(tmp_path / "add_mul" / f"input_{i}.npy").dtype == np.float16
    want = (built["inputs"][0] + built["inputs"][1]) * built["inputs"][2]
    assert np.array_equal(np.load(tmp_path / "add_mul" / "expected_0.npy"), want.numpy())


def test_reduce_models_become_row_reduce_groups(tmp_path):
    built = compile_model(AddReduce(), [TensorSpec(("M", "N"))] * 2, tmp_path / "add_reduce")
    d = descriptor(built)
    assert d["kernel_class"] == "row_reduce" and [o["op"] for o in d["body"]] == ["addf"]
    assert [l["map"] for l in d["loads"]] == [[0, 1], [0, 1]] and d["store"]["map"] == [0]

    built = compile_model(BroadcastAddReduce(), [TensorSpec(("M",)), TensorSpec(("M", "N"))], tmp_path / "bcast",
                          verify_shapes={"M": 128, "N": 16})
    d = descriptor(built)
    assert d["kernel_class"] == "row_reduce" and [l["map"] for l in d["loads"]] == [[0], [0, 1]]
    assert built["inputs"][0].shape == (128,) and built["inputs"][1].shape == (128, 16)
    assert "arg0_dim0=128" in built["shape"] and "arg1_dim1=16" in built["shape"]
    assert np.load(tmp_path / "bcast" / "expected_0.npy").shape == (128,)


def test_addmm_leaky_relu_becomes_a_matmul_group_with_fused_epilogue(tmp_path):
    specs = [TensorSpec(("M", 128), torch.bfloat16), TensorSpec((128, 64), torch.bfloat16), TensorSpec((64,), torch.bfloat16)]
    built = compile_model(LinearLeaky(), specs, tmp_path / "mm", verify_shapes={"M": 96})
    mm = descriptor(built)["matmul"]
    assert mm["epilogue"] == "BiasAddLeakyRelu" and abs(mm["alpha"] - 0.01) < 1e-9
    assert (mm["in_dtype"], mm["out_dtype"], mm["bias_dtype"]) == ("bf16", "bf16", "bf16")
    assert (mm["m"], mm["n"], mm["k"]) == ("dim_arg0_0", 64, 128)
    raw = np.load(tmp_path / "mm" / "input_0.npy")
    assert raw.dtype == np.dtype("V2") and raw.shape == (96, 128), "bf16 travels as 2-byte opaque items"
    assert build_shape_string(built["space"], built["inputs"]) == "arg0_dim0=96"


def test_scalars_views_and_broadcast_maps():
    class M(torch.nn.Module):
        def forward(self, x, col):
            return torch.relu(x * 0.5 - col) / 2.0
    text = torch_to_linalg(M(), [torch.randn(8, 16), torch.randn(8, 1)])
    assert "-> (d0, 0)>" in text, "a real unit dimension broadcasts through a constant-0 map result"
    assert "arith.constant 5.000000e-01 : f32" in text and "arith.maximumf" in text and "arith.divf" in text
    assert "tensor<8x16xf32>" in text and "?" not in text


def test_transposed_views_clamp_and_abs(tmp_path):
    class M(torch.nn.Module):
        def forward(self, a, b):
            return torch.clamp((a.t() + b).abs(), 0.1, 2.0)
    text = torch_to_linalg(M(), [torch.randn(8, 16), torch.randn(16, 8)])
    assert "-> (d1, d0)>" in text, "a.t() is a permuted indexing map, not an op"
    assert text.count("linalg.generic") == 5  # add, neg, max (abs), clamp low, clamp high
    built = compile_model(M(), [TensorSpec(("M", "N"), torch.float32), TensorSpec(("N", "M"), torch.float32)], tmp_path / "t")
    d = descriptor(built)
    assert d["kernel_class"] == "elementwise" and [l["map"] for l in d["loads"]] == [[1, 0], [0, 1]]
    assert [o["op"] for o in d["body"]] == ["addf", "subf", "maximumf", "maximumf", "minimumf"]

    class Bare(torch.nn.Module):  # a permuted output is materialised by one copy group (a bare permutation)
        def forward(self, a):
            return a.t()
    text = torch_to_linalg(Bare(), [torch.randn(4, 8)])
    assert text.count("linalg.generic") == 1 and "linalg.yield %in0" in text and "-> tensor<8x4xf32>" in text

    class Unit(torch.nn.Module):
        def forward(self, a):
            return a.unsqueeze(0)
    with pytest.raises(UnsupportedTorchOp, match="inserted unit dimensions"):
        torch_to_linalg(Unit(), [torch.randn(4, 8)])


def test_unsupported_models_are_refused():
    class Tanh(torch.nn.Module):
        def forward(self, x):
            return torch.tanh(x)
    with pytest.raises(UnsupportedTorchOp, match="tanh"):
        torch_to_linalg(Tanh(), [torch.randn(4, 4)])

    class ColSum(torch.nn.Module):
        def forward(self, x):
            return x.sum(dim=0)
    with pytest.raises(UnsupportedTorchOp, match="only the last dimension"):
        torch_to_linalg(ColSum(), [torch.randn(4, 4)])

    class WithState(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(4, 4)

        def forward(self, x):
            return self.lin(x)
    with pytest.raises(UnsupportedTorchOp, match="parameters and buffers"):
        torch_to_linalg(WithState(), [torch.randn(4, 4)])
    # the stateful entry point turns weight and bias into trailing arguments and keeps the weight as [N, K]
    from ascend_mlir_b200.torch_e2e import torch_to_linalg_with_state
    model = WithState()
    text, state = torch_to_linalg_with_state(model, [torch.randn(6, 4)])
    assert [n for n, _ in state] == ["lin.weight", "lin.bias"] and state[0][1].shape == (4, 4)
    assert "func.func @forward(%arg0: tensor<6x4xf32>, %arg1: tensor<4x4xf32>, %arg2: tensor<4xf32>)" in text
    assert "linalg.matmul_transpose_b ins(%arg0, %arg1 : tensor<6x4xf32>, tensor<4x4xf32>)" in text

    class Mixed(torch.nn.Module):
        def forward(self, a, b):
            return a + b
    with pytest.raises(UnsupportedTorchOp, match="mixed element types"):
        torch_to_linalg(Mixed(), [torch.randn(4, dtype=torch.float16), torch.randn(4, dtype=torch.float32)])


def test_transposed_weight_and_materialised_permutations():
    class MmT(torch.nn.Module):
        def forward(self, a, w):
            return torch.mm(a, w.t())
    text = torch_to_linalg(MmT(), [torch.randn(8, 16).half(), torch.randn(12, 16).half()])
    assert "linalg.matmul_transpose_b ins(%arg0, %arg1 : tensor<8x16xf16>, tensor<12x16xf16>)" in text
    assert text.count("linalg.generic") == 1  # only the rounding epilogue: no copy of the weight

    class Heads(torch.nn.Module):
        def forward(self, x):
            return x.permute(0, 2, 1, 3).contiguous()
    text = torch_to_linalg(Heads(), [torch.randn(2, 3, 4, 8)])
    assert "-> (d0, d2, d1, d3)>" in text and text.count("linalg.generic") == 1 and "tensor<2x4x3x8xf32>" in text

    class BareView(torch.nn.Module):  # a permuted output is written out by one copy group
        def forward(self, x):
            return x.transpose(0, 1)
    text = torch_to_linalg(BareView(), [torch.randn(5, 7)])
    assert text.count("linalg.generic") == 1 and "-> tensor<7x5xf32>" in text
