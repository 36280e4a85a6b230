"""Whole pipeline on the GPU for the five benchmark groups: MLIR text -> afir-opt --convert-afir-to-cuda ->
afir-translate -mlir-to-cuda (+ tiling space) -> afirt_compiler_compile -> afirt_executor_run, checked against the
oracle with the bars of the parity tests."""
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest

from ascend_mlir_b200 import build as lib_build
from ascend_mlir_b200 import configs
from ascend_mlir_b200.runtime import TilingSchema, compile_kernel
from ascend_mlir_b200.runtime.executor import CudaRuntime
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "ascend_mlir_b200" / "bin"
EXAMPLES = ROOT / "ascend_mlir_b200" / "examples"


@pytest.fixture(scope="module")
def rt():
    lib_build.build()
    r = CudaRuntime()
    r.set_device(0)
    return r


def compile_from_mlir(name, tmp_path):
    converted = tmp_path / f"{name}.converted.mlir"
    r = subprocess.run([str(BIN / "afir-opt"), "--linalg-fuse-elementwise-ops", "--mark-structured-ops", "--convert-afir-to-cuda",
                        str(EXAMPLES / f"{name}.mlir"), "-o", str(converted)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    desc, space = tmp_path / f"{name}.cuda.json", tmp_path / f"{name}.tiling_space.json"
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", str(converted), "-o", str(desc), "--tiling-space-out", str(space)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    binary = compile_kernel(desc, tmp_path / "artifact", name).read_bytes()
    return binary, json.loads(space.read_text())


def pack(space, arrays):
    """Tile parameters at their defaults, dims from the shapes of the argument arrays (shape_key arg<N>_dim<D>)."""
    values = {}
    for p in space["tiling_params"]:
        if p.get("fixed"):
            n, d = p["shape_key"][3:].split("_dim")
            values[p["name"]] = arrays[int(n)].shape[int(d)]
        else:
            values[p["name"]] = p["default"]
    return TilingSchema.from_dict(space).pack(**values)


def test_elementwise_chain_from_afir_ops(rt, tmp_path):
    binary, space = compile_from_mlir("elementwise_chain", tmp_path)
    w = configs.elementwise_chain(seed=61)  # the MLIR is static [4096, 4096]
    out = w.new_output()
    rt.run(binary, "elementwise_chain", w.inputs, [out], pack(space, w.inputs + [out]))
    assert np.array_equal(out, oracle.add_mul_f32(*w.inputs))


def test_split_group_from_linalg(rt, tmp_path):
    binary, space = compile_from_mlir("split_relu_broadcast_add_mul", tmp_path)
    w = configs.split_relu_broadcast_add_mul(seed=62)  # the MLIR is static [32, 1024, 2048]
    out = w.new_output()
    rt.run(binary, "split_relu_broadcast_add_mul", w.inputs, [out], pack(space, w.inputs + [out]))
    want = oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], 1)
    assert np.array_equal(out.view(np.uint16), want.view(np.uint16))


def test_reduce_group_from_linalg(rt, tmp_path):
    binary, space = compile_from_mlir("broadcast_add_reduce", tmp_path)
    w = configs.broadcast_add_reduce(1500, 4096, seed=63)
    out = w.new_output()
    rt.run(binary, "broadcast_add_reduce", w.inputs, [out], pack(space, w.inputs + [out]))
    _, s64, abs64 = oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1], with_bounds=True)
    assert np.all(np.abs(out - s64) <= 1e-5 * abs64)


def test_gather_group_from_linalg(rt, tmp_path):
    binary, space = compile_from_mlir("gather_elementwise", tmp_path)
    w = configs.gather_elementwise(5000, 256, 3000, seed=64)
    out = w.new_output()
    rt.run(binary, "gather_elementwise", w.inputs, [out], pack(space, w.inputs + [out]))
    assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs))


def test_transpose_group_from_linalg(rt, tmp_path):
    binary, space = compile_from_mlir("transpose_2d", tmp_path)
    assert {p["name"] for p in space["tiling_params"] if not p.get("fixed")} >= {"WARP_ROWS", "VARIANT"}
    x = np.random.default_rng(66).standard_normal((1000, 520)).astype(np.float16)
    out = np.zeros((520, 1000), np.float16)
    rt.run(binary, "transpose_2d", [x], [out], pack(space, [x, out]))
    assert out.tobytes() == oracle.transpose_2d(x).tobytes()


def test_transposed_operand_group_from_linalg(rt, tmp_path):
    binary, space = compile_from_mlir("transposed_add", tmp_path)
    rng = np.random.default_rng(67)
    a = rng.standard_normal((520, 264)).astype(np.float16)
    b = rng.standard_normal((264, 520)).astype(np.float16)
    out = np.zeros((264, 520), np.float16)
    rt.run(binary, "transposed_add", [a, b], [out], pack(space, [a, b, out]))
    assert out.tobytes() == (a.T + b).astype(np.float16).tobytes()


def test_matmul_group_from_linalg(rt, tmp_path):
    binary, space = compile_from_mlir("matmul_add_leakyrelu", tmp_path)
    w = configs.matmul_add_leakyrelu(512, 768, 320, seed=65)
    out = w.new_output()
    rt.run(binary, "matmul_add_leakyrelu", w.inputs, [out], pack(space, w.inputs + [out]))
    got = oracle.bf16_to_f32(out)
    want = oracle.bf16_to_f32(oracle.matmul_bias_leakyrelu_bf16(*w.inputs, 0.01))
    assert np.all(np.abs(got - want) <= 1e-2 * np.abs(want) + 1e-3)
