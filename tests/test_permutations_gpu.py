"""Standalone permutation groups of rank three and four (the reference accepts a bare transpose generic of any rank,
lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:775-826): MLIR text -> afir-opt -> afir-translate ->
afirt_compiler_compile -> afirt_executor_run, bit-exact against numpy's transpose.  Rank-two permutations take the
transpose kernel and are covered by the parity tests; here the permuted view is walked by the elementwise
kernels, and dims that are left above the kernels' three are walked by the launcher."""
import itertools
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest

from ascend_mlir_b200 import build as lib_build
from ascend_mlir_b200.runtime import TilingSchema, compile_kernel
from ascend_mlir_b200.runtime.executor import CudaRuntime

pytestmark = pytest.mark.gpu
BIN = Path(__file__).resolve().parent.parent / "ascend_mlir_b200" / "bin"
PASSES = ["--afir-shape-inference", "--linalg-fuse-elementwise-ops", "--mark-structured-ops", "--convert-afir-to-cuda"]
NP = {"f16": np.float16, "f32": np.float32, "i32": np.int32}


def permutation_mlir(perm, out_shape, dtype):
    """out[d0, d1, ...] = in[d_perm[0], d_perm[1], ...]"""
    rank = len(perm)
    in_shape = [out_shape[p] for p in perm]
    tensor = lambda s: "tensor<" + "x".join(map(str, s)) + f"x{dtype}>"
    dims = ", ".join(f"d{i}" for i in range(rank))
    return in_shape, f"""#in = affine_map<({dims}) -> ({", ".join(f"d{p}" for p in perm)})>
#out = affine_map<({dims}) -> ({dims})>
module {{
  func.func @permute(%x: {tensor(in_shape)}) -> {tensor(out_shape)} {{
    %e = tensor.empty() : {tensor(out_shape)}
    %t = linalg.generic {{indexing_maps = [#in, #out], iterator_types = [{", ".join(['"parallel"'] * rank)}]}}
        ins(%x : {tensor(in_shape)}) outs(%e : {tensor(out_shape)}) {{
    ^bb0(%v: {dtype}, %o: {dtype}):
      linalg.yield %v : {dtype}
    }} -> {tensor(out_shape)}
    return %t : {tensor(out_shape)}
  }}
}}
"""


@pytest.fixture(scope="module")
def rt():
    lib_build.build()
    r = CudaRuntime()
    r.set_device(0)
    return r


def run_permutation(rt, tmp_path, perm, out_shape, dtype):
    in_shape, text = permutation_mlir(perm, out_shape, dtype)
    src, conv = tmp_path / "p.mlir", tmp_path / "p.converted.mlir"
    desc, space = tmp_path / "p.cuda.json", tmp_path / "p.tiling_space.json"
    src.write_text(text)
    r = subprocess.run([str(BIN / "afir-opt"), *PASSES, str(src), "-o", str(conv)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", str(conv), "-o", str(desc), "--tiling-space-out", str(space)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    binary = compile_kernel(desc, tmp_path / "artifact", "permute").read_bytes()
    schema = json.loads(space.read_text())
    values = {p["name"]: p["default"] for p in schema["tiling_params"] if not p.get("fixed")}
    assert all(not p.get("fixed") for p in schema["tiling_params"]), "static shapes leave no dim parameters"
    rng = np.random.default_rng(sum(out_shape) + 31 * sum(i * p for i, p in enumerate(perm)))
    count = int(np.prod(in_shape))
    x = (rng.integers(-2**31, 2**31 - 1, count).astype(np.int32) if dtype == "i32"
         else rng.standard_normal(count).astype(NP[dtype])).reshape(in_shape)
    out = np.zeros(out_shape, NP[dtype])
    rt.run(binary, "permute", [x], [out], TilingSchema.from_dict(schema).pack(**values))
    want = np.ascontiguousarray(np.transpose(x, np.argsort(perm)))
    assert out.tobytes() == want.tobytes(), f"perm {perm} shape {out_shape} {dtype}"
    return rt.last_launch_count


@pytest.mark.parametrize("perm", [p for p in itertools.permutations(range(3)) if p != (0, 1, 2)])
@pytest.mark.parametrize("out_shape,dtype", [([6, 10, 14], "f16"), ([33, 72, 136], "f16"), ([17, 40, 24], "f32"), ([5, 9, 13], "i32")])
def test_every_rank_three_permutation(rt, tmp_path, perm, out_shape, dtype):
    run_permutation(rt, tmp_path, perm, out_shape, dtype)


@pytest.mark.parametrize("perm", [(0, 1, 3, 2), (0, 2, 1, 3), (1, 0, 2, 3), (3, 2, 1, 0), (2, 3, 0, 1), (1, 3, 0, 2), (3, 0, 2, 1)])
@pytest.mark.parametrize("out_shape,dtype", [([3, 5, 16, 24], "f16"), ([4, 6, 10, 14], "f32")])
def test_rank_four_permutations_with_outer_dims_walked_by_the_launcher(rt, tmp_path, perm, out_shape, dtype):
    run_permutation(rt, tmp_path, perm, out_shape, dtype)


def test_rank_five_permutation(rt, tmp_path):
    run_permutation(rt, tmp_path, (4, 2, 0, 3, 1), [2, 3, 4, 5, 8], "f16")


def test_attention_style_permutation_is_one_launch(rt, tmp_path):
    """out[b, h, s, d] = in[b, s, h, d] keeps four dims after collapsing; its views are contiguous along d, so the
    batch dim rides in the grid's second dimension instead of costing one launch per batch."""
    assert run_permutation(rt, tmp_path, (0, 2, 1, 3), [5, 6, 40, 64], "f16") == 1
    assert run_permutation(rt, tmp_path, (0, 2, 1, 3), [3, 4, 7, 9], "f32") == 1       # unaligned: the element kernel, still one launch
    assert run_permutation(rt, tmp_path, (2, 0, 3, 1), [3, 4, 8, 16], "f16") > 1        # a transposed inner pair: walked per index
