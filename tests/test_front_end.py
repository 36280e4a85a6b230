"""afir-opt / afir-translate on CPU: the five benchmark groups written as MLIR text translate to the descriptors the
kernels expect, annotation passes add the attributes the reference's FileCheck tests look for
(test/Conversion/mark-structured-ops.mlir, annotate-ascendc-kernel-kind.mlir, annotate-mix-matmul-semantics.mlir),
and anything outside the supported subset fails loudly."""
import json
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

from ascend_mlir_b200 import build as lib_build
from ascend_mlir_b200 import descriptors

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "ascend_mlir_b200" / "bin"
EXAMPLES = ROOT / "ascend_mlir_b200" / "examples"
# The reference project's examples/ directory, when a checkout is at hand (AFIR_REFERENCE_EXAMPLES); the cases that
# read it are skipped otherwise.
REFERENCE = Path(os.environ.get("AFIR_REFERENCE_EXAMPLES", "")) if os.environ.get("AFIR_REFERENCE_EXAMPLES") else None


@pytest.fixture(scope="module", autouse=True)
def built():
    lib_build.build()


def opt(*args, stdin=None):
    return subprocess.run([str(BIN / "afir-opt"), *map(str, args)], capture_output=True, text=True, input=stdin)


def translate(path, *extra):
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", str(path), *map(str, extra)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return json.loads(r.stdout) if r.stdout.strip() else None


def body_of(d):
    return [(o["op"], o["a"], o["b"]) for o in d.get("body", [])]


def views_of(d):
    return [(v["arg"], v.get("map"), v.get("offset")) for v in d["loads"]]


@pytest.mark.parametrize("name,builder", [
    ("elementwise_chain", lambda: descriptors.add_mul("f32")),
    ("split_relu_broadcast_add_mul", lambda: descriptors.split_relu_bias_mul(1)),
    ("broadcast_add_reduce", lambda: descriptors.bcast_add_rowsum("f32")),
    ("gather_elementwise", lambda: descriptors.gather_rows_scale_resid()),
    ("transpose_2d", lambda: descriptors.transpose_2d("f16")),
])
def test_config_groups_translate_to_the_expected_descriptor(name, builder):
    got = translate(EXAMPLES / f"{name}.mlir")
    want = builder().descriptor
    assert got["format"] == "afir-cuda-launch" and got["arch"] == "sm_100a" and got["kernel"] == name
    for key in ("kernel_class", "dtype", "num_inputs", "num_outputs"):
        assert got[key] == want[key], key
    assert body_of(got) == body_of(want)
    assert [v[0] for v in views_of(got)] == [v[0] for v in views_of(want)]
    assert [v[1] for v in views_of(got)] == [v[1] for v in views_of(want)]
    assert got["store"]["arg"] == want["store"]["arg"] and got["store"]["map"] == want["store"]["map"]
    if name == "transpose_2d":
        # a bare permutation is the transpose class with that kernel's launch parameters, not an elementwise group
        assert got["launch"] == want["launch"] and [t["name"] for t in got["tiling"]] == [t["name"] for t in want["tiling"]]
    if name == "gather_elementwise":
        assert got["gather"]["axis"] == 0 and got["gather"]["indices"]["dtype"] == "i32" and got["gather"]["indices"]["arg"] == 1
    if name == "split_relu_broadcast_add_mul":
        # h1 is the same argument read at a column offset of C
        assert got["loads"][2]["offset"] == [0, 0, 1024] and "offset" not in got["loads"][0]
        assert got["domain"] == [32, 1024, 1024] and got["loads"][0]["shape"] == [32, 1024, 2048]


def test_transposed_operand_stays_one_elementwise_group_with_a_permuted_view():
    got = translate(EXAMPLES / "transposed_add.mlir")
    assert got["kernel_class"] == "elementwise" and body_of(got) == [("addf", "v0", "v1")]
    assert views_of(got) == [(0, [1, 0], None), (1, [0, 1], None)]
    assert got["domain"] == ["dim_arg1_0", "dim_arg1_1"] and got["store"]["map"] == [0, 1]


def test_afir_ops_on_dynamic_shapes_take_extents_from_the_operands(tmp_path):
    src = tmp_path / "dyn.mlir"
    src.write_text("""
module {
  func.func @dyn(%a: tensor<?x?xf32>, %b: tensor<?xf32>, %c: tensor<?x1xf32>) -> tensor<?x?xf32> {
    %s = afir.add %a, %b : (tensor<?x?xf32>, tensor<?xf32>) -> tensor<?x?xf32>
    %p = afir.mul %s, %c : (tensor<?x?xf32>, tensor<?x1xf32>) -> tensor<?x?xf32>
    return %p : tensor<?x?xf32>
  }
}
""")
    d = translate(src)
    assert d["domain"] == ["dim_arg0_0", "dim_arg0_1"]
    assert [(l["shape"], l["map"]) for l in d["loads"]] == [(["dim_arg0_0", "dim_arg0_1"], [0, 1]), (["dim_arg1_0"], [1]),
                                                            (["dim_arg2_0", 1], [0, -1])]
    assert body_of(d) == [("addf", "v0", "v1"), ("mulf", "%0", "v2")]
    fields = [t["name"] for t in d["tiling"]]
    assert fields[-4:] == ["dim_arg0_0", "dim_arg0_1", "dim_arg1_0", "dim_arg2_0"]


def test_integer_afir_ops_and_arith_integer_bodies(tmp_path):
    src = tmp_path / "ints.mlir"
    src.write_text("""
#id = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @ints(%a: tensor<4x8xi32>, %b: tensor<8xi32>, %c: tensor<4x8xi32>) -> tensor<4x8xi32> {
    %s = afir.add %a, %b : (tensor<4x8xi32>, tensor<8xi32>) -> tensor<4x8xi32>
    %e = tensor.empty() : tensor<4x8xi32>
    %r = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]}
        ins(%s, %c : tensor<4x8xi32>, tensor<4x8xi32>) outs(%e : tensor<4x8xi32>) {
    ^bb0(%x: i32, %y: i32, %o: i32):
      %m = arith.muli %x, %y : i32
      %q = arith.maxsi %m, %y : i32
      linalg.yield %q : i32
    } -> tensor<4x8xi32>
    return %r : tensor<4x8xi32>
  }
}
""")
    d = translate(src)
    assert d["kernel_class"] == "elementwise" and d["dtype"] == "i32"
    assert body_of(d) == [("addi", "v0", "v1"), ("muli", "%0", "v2"), ("maxsi", "%1", "v2")]
    assert views_of(d) == [(0, [0, 1], None), (1, [1], None), (2, [0, 1], None)]


def test_matmul_group_epilogue_and_tiling_space(tmp_path):
    out, space = tmp_path / "k.cuda.json", tmp_path / "ts.json"
    assert translate(EXAMPLES / "matmul_add_leakyrelu.mlir", "-o", out, "--tiling-space-out", space) is None
    d = json.loads(out.read_text())
    assert d["kernel_class"] == "matmul" and d["num_inputs"] == 3
    mm = d["matmul"]
    assert (mm["a"], mm["b"], mm["bias"], mm["out"]) == (0, 1, 2, 3)
    assert mm["epilogue"] == "BiasAddLeakyRelu" and abs(mm["alpha"] - 0.01) < 1e-12
    assert (mm["in_dtype"], mm["bias_dtype"], mm["out_dtype"]) == ("bf16", "bf16", "bf16")
    assert (mm["m"], mm["n"], mm["k"]) == ("dim_arg0_0", "dim_arg1_1", "dim_arg0_1")
    ts = json.loads(space.read_text())
    assert ts["kernel"] == "matmul_add_leakyrelu" and ts["soc"] == "sm_100a" and ts["kernel_file"] == "matmul_add_leakyrelu.cuda.json"
    names = [p["name"] for p in ts["tiling_params"]]
    assert names == [t["name"] for t in d["tiling"]] == ["STAGES", "dim_arg0_0", "dim_arg0_1", "dim_arg1_1"]
    fixed = {p["name"]: p["shape_key"] for p in ts["tiling_params"] if p.get("fixed")}
    assert fixed == {"dim_arg0_0": "arg0_dim0", "dim_arg0_1": "arg0_dim1", "dim_arg1_1": "arg1_dim1"}


def test_annotation_passes_add_the_reference_attributes():
    r = opt("--mark-structured-ops", "--annotate-ascendc-kernel-kind", EXAMPLES / "gather_elementwise.mlir")
    assert r.returncode == 0, r.stderr
    assert 'attributes {ascendc.kernel_kind = "vec"}' in r.stdout
    marked = [l for l in r.stdout.splitlines() if "attrs = {" in l]
    assert len(marked) == 1 and "embedding_dim = 0 : i64" in marked[0] and "gather_dim" not in r.stdout
    r = opt("--annotate-ascendc-kernel-kind", "--annotate-mix-matmul-semantics", EXAMPLES / "matmul_add_leakyrelu.mlir")
    assert r.returncode == 0, r.stderr
    for needle in ['ascendc.kernel_kind = "mix"', 'abi_matmul_epilogue_kind = "BiasAddLeakyRelu"', "abi_matmul_has_bias = true",
                   'abi_matmul_layout_a = "ND"', 'abi_matmul_op_kind = "matmul"', "abi_matmul_trans_b = false"]:
        assert needle in r.stdout, needle
    r = opt("--mark-structured-ops", EXAMPLES / "elementwise_chain.mlir")
    assert r.returncode == 0 and "gather_dim" not in r.stdout and "embedding_dim" not in r.stdout


def test_column_gather_is_marked_gather_dim():
    text = """
#cols = affine_map<(d0, d1) -> (d1)>
#full = affine_map<(d0, d1) -> (d0, d1)>
func.func @index_select(%data: tensor<?x?xf16>, %idx: tensor<?xi64>) -> tensor<?x?xf16> {
  %c0 = arith.constant 0 : index
  %m = tensor.dim %data, %c0 : tensor<?x?xf16>
  %k = tensor.dim %idx, %c0 : tensor<?xi64>
  %e = tensor.empty(%m, %k) : tensor<?x?xf16>
  %g = linalg.generic {indexing_maps = [#cols, #full], iterator_types = ["parallel", "parallel"]}
      ins(%idx : tensor<?xi64>) outs(%e : tensor<?x?xf16>) {
  ^bb0(%i: i64, %o: f16):
    %r = linalg.index 0 : index
    %c = arith.index_cast %i : i64 to index
    %v = tensor.extract %data[%r, %c] : tensor<?x?xf16>
    linalg.yield %v : f16
  } -> tensor<?x?xf16>
  return %g : tensor<?x?xf16>
}
"""
    r = opt("--mark-structured-ops", "--convert-afir-to-cuda", stdin=text)
    assert r.returncode == 0, r.stderr
    assert "attrs = {gather_dim = 1 : i64}" in r.stdout and "embedding_dim" not in r.stdout
    assert 'afir.cuda_kernel_class = "gather"' in r.stdout and "afir.cuda_launch = " in r.stdout


def test_without_passes_the_module_prints_back_unchanged():
    src = (EXAMPLES / "broadcast_add_reduce.mlir").read_text()
    r = opt(EXAMPLES / "broadcast_add_reduce.mlir")
    assert r.returncode == 0 and r.stdout == src
    r = opt("--canonicalize", "--cse", "--linalg-fuse-elementwise-ops", EXAMPLES / "broadcast_add_reduce.mlir")
    assert r.returncode == 0 and 'afir.fused_group = "row_reduce"' in r.stdout


@pytest.mark.parametrize("text,needle", [
    ("func.func @f(%a: tensor<4xf32>) -> tensor<4xf32> {\n  %0 = math.exp %a : tensor<4xf32>\n  return %0 : tensor<4xf32>\n}", "unsupported operation 'math.exp'"),
    ("func.func @f(%a: tensor<4xf32>) -> tensor<4xf32> {\n  %0 = afir.exp %a : tensor<4xf32> -> tensor<4xf32>\n  return %0 : tensor<4xf32>\n}", "outside the supported elementwise set"),
    ("func.func @f(%a: tensor<4x3xf32>, %b: tensor<5xf32>) -> tensor<4x3xf32> {\n  %0 = afir.add %a, %b : (tensor<4x3xf32>, tensor<5xf32>) -> tensor<4x3xf32>\n  return %0 : tensor<4x3xf32>\n}", "not broadcastable"),
    ("func.func @f(%a: tensor<4xf32>) -> tensor<4xf32> {\n  return %a : tensor<4xf32>\n", "unterminated region"),
])
def test_inputs_outside_the_subset_fail_loudly(text, needle):
    r = opt("--convert-afir-to-cuda", stdin=text)
    assert r.returncode == 1 and needle in r.stderr, r.stderr
    assert r.stdout == ""


def test_unknown_flags_are_errors():
    r = opt("--ascendc-vectorize-everything", EXAMPLES / "elementwise_chain.mlir")
    assert r.returncode == 1 and "Unknown command line argument" in r.stderr
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-llvmir", str(EXAMPLES / "elementwise_chain.mlir")], capture_output=True, text=True)
    assert r.returncode == 1 and "Unknown command line argument" in r.stderr


def test_afir_broadcast_follows_numpy_trailing_alignment():
    text = """func.func @bias(%x: tensor<8x16xf32>, %b: tensor<16xf32>, %c: tensor<8x1xf32>) -> tensor<8x16xf32> {
  %0 = afir.add %x, %b : (tensor<8x16xf32>, tensor<16xf32>) -> tensor<8x16xf32>
  %1 = afir.mul %0, %c : (tensor<8x16xf32>, tensor<8x1xf32>) -> tensor<8x16xf32>
  return %1 : tensor<8x16xf32>
}"""
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", "-"], capture_output=True, text=True, input=text)
    assert r.returncode == 0, r.stderr
    d = json.loads(r.stdout)
    assert [v["map"] for v in d["loads"]] == [[0, 1], [1], [0, -1]]
    assert body_of(d) == [("addf", "v0", "v1"), ("mulf", "%0", "v2")]


def test_a_string_that_never_ends_is_an_error_not_a_crash():
    """An attribute string without its closing quote (after an op name, in linalg.generic's dictionary, in an afir
    op's attributes): the tools stop with a message; found by mutating inputs."""
    cases = ["""func.func @f(%a: memref<8x8xf16>, %b: memref<8x16xf16>, %c: memref<8x16xf32>) {
  linalg.matmul {ascendc.unit = "AiCore.Cube} ins(%a, %b : memref<8x8xf16>, memref<8x16xf16>) outs(%c : memref<8x16xf32>)
  return
}""", """func.func @f(%x: tensor<4xf32>) -> tensor<4xf32> {
  %0 = afir.relu %x {note = "never closed} : tensor<4xf32> -> tensor<4xf32>
  return %0 : tensor<4xf32>
}""", """func.func @f(%s: memref<4xf32>, %d: memref<4xf32>) {
  linalg.generic {indexing_maps = [affine_map<(d0) -> (d0)>, affine_map<(d0) -> (d0)>], iterator_types = ["parallel]} ins(%s : memref<4xf32>) outs(%d : memref<4xf32>) {
  ^bb0(%x: f32, %y: f32):
    linalg.yield %x : f32
  }
  return
}"""]
    for text in cases:
        r = opt("--annotate-ascendc-kernel-kind", "-", stdin=text)
        assert r.returncode == 1 and "error: line" in r.stderr, (r.returncode, r.stderr)


def test_generics_nested_without_end_are_an_error_not_a_stack_overflow():
    opening = ('%r = linalg.generic {indexing_maps = [affine_map<(d0) -> (d0)>, affine_map<(d0) -> (d0)>], iterator_types = ["parallel"]} '
               'ins(%s : tensor<4xf32>) outs(%d : tensor<4xf32>) {\n^bb0(%x: f32, %y: f32):\n')
    text = "func.func @f(%s: tensor<4xf32>, %d: tensor<4xf32>) -> tensor<4xf32> {\n" + opening * 50000
    r = opt("-", stdin=text)
    assert r.returncode == 1 and "regions nested too deep" in r.stderr


def test_kernel_kind_follows_the_units_a_lowering_stage_assigned():
    """--annotate-ascendc-kernel-kind on buffer-level functions whose ops carry ascendc.unit (what the reference's
    test/Conversion/annotate-ascendc-kernel-kind.mlir feeds the pass): Cube only = "cube", Vector only = "vec", both =
    "mix"; the attribute may sit after the op name, in linalg.generic's dictionary or in its trailing attrs; a unit
    the rule does not know is an error; a function without units is classified from its fused group as before."""
    copy = """linalg.generic {UNIT indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
      iterator_types = ["parallel", "parallel"]} ins(%src : memref<8x16xf32>) outs(%dst : memref<8x16xf32>) TRAILING {
    ^bb0(%x: f32, %y: f32):
      linalg.yield %x : f32
    }"""
    text = f"""func.func @product(%a: memref<8x8xf16>, %b: memref<8x16xf16>, %c: memref<8x16xf32>) {{
  linalg.matmul {{ascendc.unit = "AiCore.Cube"}} ins(%a, %b : memref<8x8xf16>, memref<8x16xf16>) outs(%c : memref<8x16xf32>)
  return
}}
func.func @copy_front(%src: memref<8x16xf32>, %dst: memref<8x16xf32>) {{
  {copy.replace("UNIT", 'ascendc.unit = "AiCore.Vector",').replace("TRAILING", "")}
  return
}}
func.func @copy_trailing(%src: memref<8x16xf32>, %dst: memref<8x16xf32>) {{
  {copy.replace("UNIT", "").replace("TRAILING", 'attrs = {ascendc.unit = "AiCore.Vector"}')}
  return
}}
func.func @both(%a: memref<8x8xf16>, %b: memref<8x16xf16>, %c: memref<8x16xf32>, %src: memref<8x16xf32>, %dst: memref<8x16xf32>) {{
  linalg.matmul {{ascendc.unit = "AiCore.Cube"}} ins(%a, %b : memref<8x8xf16>, memref<8x16xf16>) outs(%c : memref<8x16xf32>)
  {copy.replace("UNIT", 'ascendc.unit = "AiCore.Vector",').replace("TRAILING", "")}
  return
}}
"""
    r = opt("--annotate-ascendc-kernel-kind", "-", stdin=text)
    assert r.returncode == 0, r.stderr
    kinds = {}
    for line in r.stdout.splitlines():
        if line.startswith("func.func @"):
            kinds[line.split("@")[1].split("(")[0]] = line.split('ascendc.kernel_kind = "')[1].split('"')[0]
    assert kinds == {"product": "cube", "copy_front": "vec", "copy_trailing": "vec", "both": "mix"}
    bad = opt("--annotate-ascendc-kernel-kind", "-", stdin=text.replace("AiCore.Cube", "AiCore.Scalar", 1))
    assert bad.returncode == 1 and "unsupported ascendc.unit value for kernel kind: AiCore.Scalar" in bad.stderr
    # tensor-level groups without units: from the group, as before
    r = opt("--annotate-ascendc-kernel-kind", EXAMPLES / "matmul_add_leakyrelu.mlir")
    assert r.returncode == 0 and 'ascendc.kernel_kind = "mix"' in r.stdout


def test_shape_inference_refines_result_types_like_the_reference_pass():
    """--afir-shape-inference on the first function of the reference's test/Dialect/AFIR/Transforms/shapeInference.mlir
    (tensor<4x1x31xf32> with tensor<1x30x1xf32>; its FileCheck line wants "-> tensor<4x30x31xf32>"): every op result,
    the operand types of the users, the return op and the function's result type carry the inferred shape."""
    text = """func.func @HashCopyAscGraph(%arg0: tensor<4x1x31xf32>, %arg1: tensor<1x30x1xf32>) -> tensor<?x?x?xf32> {
    %2 = afir.add %arg0, %arg1 : (tensor<4x1x31xf32>, tensor<1x30x1xf32>) -> tensor<?x?x?xf32>
    %3 = afir.mul %2, %arg1 : (tensor<?x?x?xf32>, tensor<1x30x1xf32>) -> tensor<?x?x?xf32>
    %4 = afir.sub %arg1, %3 : (tensor<1x30x1xf32>, tensor<?x?x?xf32>) -> tensor<?x?x?xf32>
    return %4 : tensor<?x?x?xf32>
  }
"""
    r = opt("--afir-shape-inference", "-", stdin=text)
    assert r.returncode == 0, r.stderr
    out = r.stdout
    assert out.count("-> tensor<4x30x31xf32>") == 4 and "?" not in out
    assert "%3 = afir.mul %2, %arg1 : (tensor<4x30x31xf32>, tensor<1x30x1xf32>) -> tensor<4x30x31xf32>" in out
    assert "%4 = afir.sub %arg1, %3 : (tensor<1x30x1xf32>, tensor<4x30x31xf32>) -> tensor<4x30x31xf32>" in out
    assert "return %4 : tensor<4x30x31xf32>\n  }" in out
    # a second run changes nothing
    again = opt("--afir-shape-inference", "-", stdin=out)
    assert again.returncode == 0 and again.stdout == out


def test_shape_inference_rules_for_ranks_dynamic_extents_and_conflicts():
    """Trailing alignment across ranks; a dynamic extent yields to a static one from another operand whatever the order;
    extents that stay unknown stay '?'; an op whose operands do not broadcast, or whose declared result contradicts the
    inference, keeps its types (the reference's pass skips such an op without failing)."""
    text = """func.func @ranks(%a: tensor<8x?xf16>, %b: tensor<16xf16>, %c: tensor<?x?xf16>) -> tensor<?x?xf16> {
    %0 = afir.mul %a, %b : (tensor<8x?xf16>, tensor<16xf16>) -> tensor<?x?xf16>
    %1 = afir.div %c, %0 : (tensor<?x?xf16>, tensor<?x?xf16>) -> tensor<?x?xf16>
    return %1 : tensor<?x?xf16>
}
func.func @unknown(%a: tensor<?x4xi32>, %b: tensor<?x1xi32>) -> tensor<?x?xi32> {
    %0 = afir.add %a, %b : (tensor<?x4xi32>, tensor<?x1xi32>) -> tensor<?x?xi32>
    return %0 : tensor<?x?xi32>
}
func.func @conflict(%a: tensor<8x4xf32>, %b: tensor<8x5xf32>) -> tensor<?x?xf32> {
    %0 = afir.add %a, %b : (tensor<8x4xf32>, tensor<8x5xf32>) -> tensor<?x?xf32>
    return %0 : tensor<?x?xf32>
}
func.func @contradiction(%a: tensor<8x4xf32>, %b: tensor<8x4xf32>) -> tensor<8x7xf32> {
    %0 = afir.add %a, %b : (tensor<8x4xf32>, tensor<8x4xf32>) -> tensor<8x7xf32>
    return %0 : tensor<8x7xf32>
}
"""
    r = opt("--afir-shape-inference", "-", stdin=text)
    assert r.returncode == 0, r.stderr
    out = r.stdout
    assert "%0 = afir.mul %a, %b : (tensor<8x?xf16>, tensor<16xf16>) -> tensor<8x16xf16>" in out
    assert "%1 = afir.div %c, %0 : (tensor<?x?xf16>, tensor<8x16xf16>) -> tensor<8x16xf16>" in out
    assert "@ranks(%a: tensor<8x?xf16>, %b: tensor<16xf16>, %c: tensor<?x?xf16>) -> tensor<8x16xf16> {" in out
    assert "%0 = afir.add %a, %b : (tensor<?x4xi32>, tensor<?x1xi32>) -> tensor<?x4xi32>" in out and "-> tensor<?x4xi32> {" in out
    assert "(tensor<8x4xf32>, tensor<8x5xf32>) -> tensor<?x?xf32>" in out and "return %0 : tensor<?x?xf32>" in out
    assert "(tensor<8x4xf32>, tensor<8x4xf32>) -> tensor<8x7xf32>" in out


def test_wider_afir_elementwise_family_lowers_to_the_fused_body_ops(tmp_path):
    """afir.relu / leaky_relu / maximum / minimum / truediv / clip_by_value (include/Dialect/AFIR/Ops/Basic/math.td:60-121):
    unary ops print "T -> R", leaky_relu carries negative_slop; relu = max(x, 0), leaky_relu = max(x, slope * x) with the
    slope as an f32, clip_by_value = min(max(x, low), high); shapes broadcast like add / mul.  The second function is
    the clip case of the reference's shapeInference.mlir, whose FileCheck line wants "-> tensor<4x20x32xf32>"."""
    text = """func.func @act(%x: tensor<?x64xf16>, %y: tensor<64xf16>) -> tensor<?x?xf16> {
    %0 = afir.relu %x : tensor<?x64xf16> -> tensor<?x?xf16>
    %1 = afir.leaky_relu %0 {negative_slop = 0.01 : f32} : tensor<?x?xf16> -> tensor<?x?xf16>
    %2 = afir.maximum %1, %y : (tensor<?x?xf16>, tensor<64xf16>) -> tensor<?x?xf16>
    %3 = afir.truediv %2, %y : (tensor<?x?xf16>, tensor<64xf16>) -> tensor<?x?xf16>
    %4 = afir.minimum %3, %x : (tensor<?x?xf16>, tensor<?x64xf16>) -> tensor<?x?xf16>
    return %4 : tensor<?x?xf16>
}
func.func @test_clip_by_value(%arg0: tensor<4x1x1xf32>, %arg1: tensor<1x20x1xf32>, %arg2: tensor<1x1x32xf32>) -> tensor<?x?x?xf32> {
    %0 = afir.clip_by_value %arg0, %arg1, %arg2 : (tensor<4x1x1xf32>, tensor<1x20x1xf32>, tensor<1x1x32xf32>) -> tensor<?x?x?xf32>
    return %0 : tensor<?x?x?xf32>
}
"""
    src = tmp_path / "family.mlir"
    src.write_text(text)
    r = opt("--afir-shape-inference", src)
    assert r.returncode == 0, r.stderr
    assert "%0 = afir.relu %x : tensor<?x64xf16> -> tensor<?x64xf16>" in r.stdout  # the unary form keeps its bare operand type
    assert "%1 = afir.leaky_relu %0 {negative_slop = 0.01 : f32} : tensor<?x64xf16> -> tensor<?x64xf16>" in r.stdout
    assert "-> tensor<4x20x32xf32> {" in r.stdout and r.stdout.count("-> tensor<4x20x32xf32>") == 2
    act = translate(src, "--function", "act")
    slope = float(np.float32(0.01))
    assert act["kernel_class"] == "elementwise" and act["dtype"] == "f16" and act["domain"] == ["dim_arg0_0", 64]
    assert body_of(act) == [("maximumf", "v0", 0.0), ("mulf", "%0", slope), ("maximumf", "%0", "%1"), ("maximumf", "%2", "v1"),
                            ("divf", "%3", "v1"), ("minimumf", "%4", "v0")]
    assert [v["map"] for v in act["loads"]] == [[0, 1], [1]]
    clip = translate(src, "--function", "test_clip_by_value")
    assert clip["domain"] == [4, 20, 32] and body_of(clip) == [("maximumf", "v0", "v1"), ("minimumf", "%0", "v2")]
    assert [v["map"] for v in clip["loads"]] == [[0, -1, -1], [-1, 1, -1], [-1, -1, 2]]
    # the group's kernel is generated and compiles for sm_100a
    cubin = tmp_path / "act.cubin"
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda-kernel", str(src), "--function", "act", "-o", str(tmp_path / "act.cu"),
                        "--cubin-out", str(cubin)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert cubin.read_bytes()[:4] == b"\x7fELF" and "P::max(r0, r1)" in (tmp_path / "act.cu").read_text()
    # afir.neg: x * -1 on floats (exact, zeros and infinities included), 0 - x on integers (wraps like the type)
    for elem, want in (("f32", [("mulf", "v0", -1.0)]), ("i32", [("subi", 0, "v0")])):
        neg = f"func.func @n(%x: tensor<8x?x{elem}>) -> tensor<8x?x{elem}> {{\n  %0 = afir.neg %x : tensor<8x?x{elem}> -> tensor<8x?x{elem}>\n  return %0 : tensor<8x?x{elem}>\n}}\n"
        r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", "-"], capture_output=True, text=True, input=neg)
        assert r.returncode == 0, r.stderr
        assert body_of(json.loads(r.stdout)) == want
    # afir.abs: max(x, x * -1)
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", "-"], capture_output=True, text=True,
                       input="func.func @a(%x: tensor<?x8xf16>) -> tensor<?x8xf16> {\n  %0 = afir.abs %x : tensor<?x8xf16> -> tensor<?x8xf16>\n  return %0 : tensor<?x8xf16>\n}\n")
    assert r.returncode == 0 and body_of(json.loads(r.stdout)) == [("mulf", "v0", -1.0), ("maximumf", "v0", "%0")], r.stderr
    # what stays outside: a slope the max form does not express, an op of the family with no body op, wrong arity
    for bad, needle in [(text.replace("0.01 : f32", "1.5 : f32"), "negative_slop outside [0, 1]"),
                        (text.replace("afir.relu %x :", "afir.exp %x :"), "outside the supported elementwise set"),
                        (text.replace("{negative_slop = 0.01 : f32} ", ""), "needs its negative_slop attribute"),
                        (text.replace("afir.maximum %1, %y :", "afir.maximum %1 :"), "takes 2 operands")]:
        r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", "-", "--function", "act"], capture_output=True, text=True, input=bad)
        assert r.returncode == 1 and needle in r.stderr, (needle, r.stderr)


def test_afir_concat_infers_like_the_reference_and_lowers_to_row_ranges_of_one_output(tmp_path):
    """afir.concat (concat_axis in its attributes, "T, U -> R" type form).  Shapes as in the reference's shapeInference.mlir
    (2x4, 3x4, 4x4 along axis 0: its FileCheck line wants "-> tensor<9x4xf32>"; a concat of a concat along axis 1), and a
    concat along axis 0 of two elementwise chains becomes one kernel of two groups that write their own row ranges."""
    text = """func.func @test_concat(%arg0: tensor<2x4xf32>, %arg1: tensor<3x4xf32>, %arg2: tensor<4x4xf32>) -> tensor<?x?xf32> {
  %0 = afir.concat %arg0, %arg1, %arg2 {concat_axis = 0 : i32} : tensor<2x4xf32>, tensor<3x4xf32>, tensor<4x4xf32> -> tensor<?x?xf32>
  return %0 : tensor<?x?xf32>
}
func.func @two(%arg0: tensor<2x4xf32>, %arg1: tensor<2x4xf32>, %arg2: tensor<4x4xf32>) -> tensor<?x?xf32> {
  %0 = afir.concat %arg0, %arg1 {concat_axis = 0 : i32} : tensor<2x4xf32>, tensor<2x4xf32> -> tensor<?x?xf32>
  %1 = afir.concat %0, %arg2 {concat_axis = 1 : i32} : tensor<?x?xf32>, tensor<4x4xf32> -> tensor<?x?xf32>
  return %1 : tensor<?x?xf32>
}
func.func @halves(%a: tensor<?x64xf16>, %b: tensor<?x64xf16>, %s: tensor<64xf16>) -> tensor<?x?xf16> {
  %0 = afir.relu %a : tensor<?x64xf16> -> tensor<?x?xf16>
  %1 = afir.mul %b, %s : (tensor<?x64xf16>, tensor<64xf16>) -> tensor<?x?xf16>
  %2 = afir.concat %0, %1 {concat_axis = 0 : i32} : tensor<?x?xf16>, tensor<?x?xf16> -> tensor<?x?xf16>
  return %2 : tensor<?x?xf16>
}
"""
    src = tmp_path / "concat.mlir"
    src.write_text(text)
    out = opt("--afir-shape-inference", src).stdout
    assert "tensor<2x4xf32>, tensor<3x4xf32>, tensor<4x4xf32> -> tensor<9x4xf32>" in out and "@test_concat(" in out and "-> tensor<9x4xf32> {" in out
    assert "%0 = afir.concat %arg0, %arg1 {concat_axis = 0 : i32} : tensor<2x4xf32>, tensor<2x4xf32> -> tensor<4x4xf32>" in out
    assert "%1 = afir.concat %0, %arg2 {concat_axis = 1 : i32} : tensor<4x4xf32>, tensor<4x4xf32> -> tensor<4x8xf32>" in out
    assert "%2 = afir.concat %0, %1 {concat_axis = 0 : i32} : tensor<?x64xf16>, tensor<?x64xf16> -> tensor<?x64xf16>" in out  # dynamic rows stay dynamic
    d = translate(src, "--function", "halves")
    assert d["kernel_class"] == "elementwise" and len(d["groups"]) == 2
    first, second = d["groups"]
    assert body_of(first) == [("maximumf", "v0", 0.0)] and body_of(second) == [("mulf", "v0", "v1")]
    assert first["store"]["arg"] == second["store"]["arg"] == 3 and "offset" not in first["store"]
    assert second["store"]["offset"] == ["dim_arg0_0", 0]  # the second half starts where the first ends
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", str(src), "--function", "two"], capture_output=True, text=True)
    assert r.returncode == 1 and "only concatenation along dim 0 is supported" in r.stderr
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", "-"], capture_output=True, text=True,
                       input=text.replace("{concat_axis = 0 : i32} : tensor<2x4xf32>, tensor<3x4xf32>", "{} : tensor<2x4xf32>, tensor<3x4xf32>"))
    assert r.returncode == 1 and "needs its concat_axis attribute" in r.stderr


def test_afir_reductions_infer_their_shape_and_a_last_axis_sum_is_the_row_reduction(tmp_path):
    """The afir reductions (reduce.td:43-49) drop their axis (the max case of the reference's shapeInference.mlir: a
    4x5 input gives "-> tensor<5xf16>" along axis 0 and "-> tensor<4xf16>" along axis 1, two results, both carried to the
    return op and the function type; `axis` is told apart from vectorized_axis).  afir.add with a column operand followed
    by afir.sum along the last axis is the broadcast-add-reduce group: same descriptor as its linalg form."""
    text = """func.func @test_max_reduce_f16(%arg0: tensor<4x5xf16>) -> (tensor<?xf16>, tensor<?xf16>) {
  %0 = afir.max %arg0 {vectorized_axis = [0], axis = 0 : i32} : tensor<4x5xf16> -> tensor<?xf16>
  %1 = afir.max %arg0 {axis = 1 : i32} : tensor<4x5xf16> -> tensor<?xf16>
  return %0, %1 : tensor<?xf16>, tensor<?xf16>
}
func.func @broadcast_add_reduce(%a: tensor<?x1xf32>, %b: tensor<?x?xf32>) -> tensor<?xf32> {
  %0 = afir.add %a, %b : (tensor<?x1xf32>, tensor<?x?xf32>) -> tensor<?x?xf32>
  %1 = afir.sum %0 {axis = 1 : i32} : tensor<?x?xf32> -> tensor<?xf32>
  return %1 : tensor<?xf32>
}
"""
    src = tmp_path / "reduce.mlir"
    src.write_text(text)
    out = opt("--afir-shape-inference", src).stdout
    assert "-> (tensor<5xf16>, tensor<4xf16>) {" in out and "return %0, %1 : tensor<5xf16>, tensor<4xf16>" in out
    assert "axis = 0 : i32} : tensor<4x5xf16> -> tensor<5xf16>" in out and "{axis = 1 : i32} : tensor<4x5xf16> -> tensor<4xf16>" in out
    got = translate(src, "--function", "broadcast_add_reduce")
    want = translate(EXAMPLES / "broadcast_add_reduce.mlir")
    assert got["kernel_class"] == want["kernel_class"] == "row_reduce"
    assert body_of(got) == body_of(want) == [("addf", "v0", "v1")]
    assert [(v["arg"], v["map"][0]) for v in got["loads"]] == [(v["arg"], v["map"][0]) for v in want["loads"]] == [(0, 0), (1, 0)]
    assert got["store"]["arg"] == want["store"]["arg"] == 2 and got["tiling"][:6] == want["tiling"][:6]
    # a kernel is generated for it (the staged and the finalize entries beside the main one) and compiles
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda-kernel", str(src), "--function", "broadcast_add_reduce",
                        "-o", str(tmp_path / "k.cu"), "--cubin-out", str(tmp_path / "k.cubin")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert (tmp_path / "k.cubin").read_bytes()[:4] == b"\x7fELF" and "broadcast_add_reduce__staged" in (tmp_path / "k.cu").read_text()
    for bad, needle in [(text.replace("afir.sum %0 {axis = 1", "afir.sum %0 {axis = 0"), "only a sum along the last axis is lowered"),
                        (text.replace("afir.sum %0 {axis = 1 : i32}", "afir.sum %0 {vectorized_axis = [0]}"), "needs its axis attribute"),
                        (text.replace("afir.sum", "afir.mean"), "only afir.sum is lowered")]:
        r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", "-", "--function", "broadcast_add_reduce"],
                           capture_output=True, text=True, input=bad)
        assert r.returncode == 1 and needle in r.stderr, (needle, r.stderr)


def test_shape_inference_before_the_conversion_gives_literal_extents(tmp_path):
    src = tmp_path / "chain.mlir"
    src.write_text("""func.func @chain(%a: tensor<64x1xf32>, %b: tensor<1x256xf32>) -> tensor<?x?xf32> {
  %0 = afir.add %a, %b : (tensor<64x1xf32>, tensor<1x256xf32>) -> tensor<?x?xf32>
  %1 = afir.mul %0, %b : (tensor<?x?xf32>, tensor<1x256xf32>) -> tensor<?x?xf32>
  return %1 : tensor<?x?xf32>
}
""")
    refined = tmp_path / "refined.mlir"
    r = opt("--afir-shape-inference", src, "-o", refined)
    assert r.returncode == 0, r.stderr
    assert "-> tensor<64x256xf32> {" in refined.read_text()
    d = translate(refined)
    assert d["kernel_class"] == "elementwise" and d["domain"] == [64, 256]
    assert [v["map"] for v in d["loads"]] == [[0, -1], [-1, 1]] and body_of(d) == [("addf", "v0", "v1"), ("mulf", "%0", "v1")]


@pytest.mark.skipif(REFERENCE is None or not REFERENCE.exists(), reason="AFIR_REFERENCE_EXAMPLES does not name the reference's examples/")
@pytest.mark.parametrize("example,cls", [("add-broadcast-concat", "elementwise"), ("broadcast-add-reduce", "row_reduce"),
                                         ("gather-elementwise-fusion", "gather"), ("matmul-add-leakyrelu", "matmul"),
                                         ("relu-broadcast-transpose", "elementwise"), ("split-relu-brc-add-mul", "elementwise")])
def test_reference_example_inputs_translate(example, cls):
    d = translate(REFERENCE / example / "step0_input.mlir")
    assert d["kernel_class"] == cls
    if example == "matmul-add-leakyrelu":
        assert d["matmul"]["epilogue"] == "BiasAddLeakyRelu" and abs(d["matmul"]["alpha"] - 0.001) < 1e-12
        assert (d["matmul"]["in_dtype"], d["matmul"]["out_dtype"], d["matmul"]["bias_dtype"]) == ("f16", "f32", "f32")
    if example == "gather-elementwise-fusion":
        assert d["gather"]["axis"] == 1 and body_of(d) == [("maximumf", "v0", 0.0), ("addf", "%0", "v1")]
    if example in ("add-broadcast-concat", "split-relu-brc-add-mul"):
        assert len(d["groups"]) == 2 and d["groups"][1]["store"]["offset"][0] != 0


def test_mutated_inputs_are_rejected_or_accepted_but_never_crash_the_tools():
    """Seeded text mutations (deleted spans, duplicated spans, swapped characters, stray brackets) of the example
    modules: afir-opt and afir-translate must answer with exit code 0 or 1 and, on 1, an 'error:' line."""
    import random
    rng = random.Random(20240607)
    sources = [(EXAMPLES / n).read_text() for n in ("broadcast_add_reduce.mlir", "matmul_add_leakyrelu.mlir",
                                                     "gather_elementwise.mlir", "split_relu_broadcast_add_mul.mlir")]
    crashes = []
    for trial in range(160):
        text = sources[trial % len(sources)]
        for _ in range(rng.randint(1, 3)):
            i = rng.randrange(len(text))
            kind = rng.randrange(4)
            if kind == 0:
                text = text[:i] + text[i + rng.randint(1, 12):]
            elif kind == 1:
                j = min(len(text), i + rng.randint(1, 20))
                text = text[:j] + text[i:j] + text[j:]
            elif kind == 2 and i + 1 < len(text):
                text = text[:i] + text[i + 1] + text[i] + text[i + 2:]
            else:
                text = text[:i] + rng.choice("{}()<>[]%#:,") + text[i:]
        r = subprocess.run([str(BIN / "afir-opt"), "--mark-structured-ops", "--convert-afir-to-cuda", "-"], input=text,
                           capture_output=True, text=True)
        if r.returncode not in (0, 1) or (r.returncode == 1 and "error" not in r.stderr.lower()):
            crashes.append((trial, r.returncode, r.stderr[-200:]))
            continue
        if r.returncode == 0:
            t = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda", "-"], input=r.stdout, capture_output=True, text=True)
            if t.returncode not in (0, 1) or (t.returncode == 1 and "error" not in t.stderr.lower()):
                crashes.append((trial, "translate", t.returncode, t.stderr[-200:]))
    assert not crashes, crashes[:5]


def test_permutation_of_rank_five_is_an_elementwise_group_with_a_permuted_view(tmp_path):
    """The reference takes a bare transpose generic of any rank (ComputeConversion.cpp:775-826); only rank two has
    a kernel class of its own here, the others read the input through its permuted view."""
    from test_permutations_gpu import permutation_mlir
    from ascend_mlir_b200.runtime import compile_kernel
    perm, out_shape = (4, 2, 0, 3, 1), [2, 3, 4, 5, 8]
    in_shape, text = permutation_mlir(perm, out_shape, "f16")
    src = tmp_path / "p.mlir"
    src.write_text(text)
    got = translate(src)
    assert got["kernel_class"] == "elementwise" and body_of(got) == []
    assert got["domain"] == out_shape and got["store"]["map"] == [0, 1, 2, 3, 4]
    assert views_of(got) == [(0, list(perm), None)] and got["loads"][0]["shape"] == in_shape
    desc = tmp_path / "p.cuda.json"
    desc.write_text(json.dumps(got))
    assert compile_kernel(desc, tmp_path / "artifact", "permute").exists()  # the descriptor parser takes up to eight dims


def test_matmul_transpose_b_sets_the_abi_attribute_and_the_descriptor_flag(tmp_path):
    """The reference's matmul ABI carries abi_matmul_trans_b (always false there: AnnotateMixMatmulSemanticsPass);
    linalg.matmul_transpose_b sets it, and the descriptor asks the kernel for B as [N, K]."""
    src = tmp_path / "mmt.mlir"
    src.write_text("""#bias = affine_map<(d0, d1) -> (d1)>
#id = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @linear(%x: tensor<64x128xbf16>, %w: tensor<256x128xbf16>, %b: tensor<256xbf16>) -> tensor<64x256xbf16> {
    %zero = arith.constant 0.0 : f32
    %e = tensor.empty() : tensor<64x256xf32>
    %init = linalg.fill ins(%zero : f32) outs(%e : tensor<64x256xf32>) -> tensor<64x256xf32>
    %mm = linalg.matmul_transpose_b ins(%x, %w : tensor<64x128xbf16>, tensor<256x128xbf16>) outs(%init : tensor<64x256xf32>) -> tensor<64x256xf32>
    %o = tensor.empty() : tensor<64x256xbf16>
    %r = linalg.generic {indexing_maps = [#id, #bias, #id], iterator_types = ["parallel", "parallel"]}
        ins(%mm, %b : tensor<64x256xf32>, tensor<256xbf16>) outs(%o : tensor<64x256xbf16>) {
    ^bb0(%acc: f32, %bv: bf16, %out: bf16):
      %bf = arith.extf %bv : bf16 to f32
      %s = arith.addf %acc, %bf : f32
      %t = arith.truncf %s : f32 to bf16
      linalg.yield %t : bf16
    } -> tensor<64x256xbf16>
    return %r : tensor<64x256xbf16>
  }
}
""")
    got = translate(src)
    mm = got["matmul"]
    assert got["kernel_class"] == "matmul" and mm["transpose_b"] is True and mm["epilogue"] == "BiasAdd"
    assert (mm["m"], mm["n"], mm["k"]) == (64, 256, 128) and (mm["a"], mm["b"], mm["bias"]) == (0, 1, 2)
    converted = tmp_path / "mmt.converted.mlir"
    r = subprocess.run([str(BIN / "afir-opt"), "--annotate-ascendc-kernel-kind", "--annotate-mix-matmul-semantics", str(src), "-o", str(converted)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert "abi_matmul_trans_b = true" in converted.read_text() and "abi_matmul_trans_a = false" in converted.read_text()


# ---- the reference's stage names and schedule files --------------------------------------------------------------------
REFERENCE_STAGES = [
    [],                                      # stage 0: parse only
    ["--linalg-fuse-elementwise-ops"],
    ["--transform-interpreter", "--canonicalize", "--cse"],
    ["--one-shot-bufferize=bufferize-function-boundaries=true allow-return-allocs-from-loops=true "
     "function-boundary-type-conversion=identity-layout-map", "--cse"],
    ["--ascendc-buffer-placement"],
    ["--linalg-to-ascendc", "--canonicalize", "--cse"],
    ["--ascendc-parallelize", "--canonicalize", "--cse"],
    ["--ascendc-prepare-for-emit", "--canonicalize", "--cse"],
    ["--canonicalize-cann-signature"],
]


def run_reference_stages(src, work):
    """The command lines of the reference's examples/*/run.sh and python/torch/framework/pipeline.py:_run_mlir_pipeline,
    stage by stage, each reading the previous stage's file; returns the last file."""
    for i, flags in enumerate(REFERENCE_STAGES):
        dst = work / f"stage{i}.mlir"
        r = opt(*flags, src, "-o", dst)
        assert r.returncode == 0, (flags, r.stderr)
        src = dst
    return src


def test_reference_stage_names_drive_the_tools_end_to_end(tmp_path):
    from ascend_mlir_b200.runtime.compiler import compile_kernel
    last = run_reference_stages(EXAMPLES / "broadcast_add_reduce_scheduled.mlir", tmp_path)
    text = last.read_text()
    # the schedule was read (three index arguments, two tilings, two annotations) and then removed with its module attribute
    assert "afir.tile_index_args = 3 : i64" in text
    assert 'afir.tile_sizes = "[[%rows_per_group, 0], [%rows_per_step, %cols_per_step]]"' in text
    assert 'afir.schedule_annotations = ["ascendc.parallel", "ascendc.unit"]' in text
    assert "transform.named_sequence" not in text and "transform.with_named_sequence" not in text
    assert "transform.named_sequence" in (tmp_path / "stage7.mlir").read_text()  # kept until the signature stage
    assert "cann.num_inputs = 2 : i64" in text and "cann.num_outputs = 1 : i64" in text
    for stage in ("one_shot_bufferize", "ascendc_buffer_placement", "linalg_to_ascendc", "ascendc_parallelize", "ascendc_prepare_for_emit"):
        assert f"afir.stage.{stage} = true" in text
    # stage 8 under the reference's flag name: a kernel SOURCE file that carries its launch descriptor
    kernel_cpp, space = tmp_path / "step8_kernel.cpp", tmp_path / "step8_kernel.tiling_space.json"
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cann", str(last), "-o", str(kernel_cpp), "--tiling-space-out", str(space)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    source = kernel_cpp.read_text()
    assert source.startswith("// afir-cuda-launch-descriptor-begin\n// {")
    assert 'extern "C" __global__ void __launch_bounds__(512) broadcast_add_reduce_scheduled(const void *arg0, const void *arg1, void *arg2, ' in source
    assert json.loads(space.read_text())["kernel"] == "broadcast_add_reduce_scheduled"
    # ... which is what the compile step takes: that very text is compiled for sm_100a
    blob = compile_kernel(kernel_cpp, tmp_path / "artifact", "broadcast_add_reduce_scheduled").read_bytes()
    assert blob[:4] == b"AFCU" and int.from_bytes(blob[4:8], "little") == 2
    json_len = int.from_bytes(blob[8:12], "little")
    assert json.loads(blob[12:12 + json_len])["kernel_class"] == "row_reduce"
    off = 12 + json_len
    cubin_len = int.from_bytes(blob[off:off + 4], "little")
    assert blob[off + 4:off + 8] == b"\x7fELF"
    off += 4 + cubin_len
    source_len = int.from_bytes(blob[off:off + 4], "little")
    assert blob[off + 4:off + 4 + source_len].decode() == source


def test_transform_interpreter_needs_a_schedule_and_checks_it(tmp_path):
    r = opt("--transform-interpreter", EXAMPLES / "broadcast_add_reduce.mlir")
    assert r.returncode == 1 and "holds no transform.named_sequence" in r.stderr
    bad = (EXAMPLES / "broadcast_add_reduce_scheduled.mlir").read_text().replace("add_index_args %func, 3", "add_index_args %func, 0")
    r = opt("--transform-interpreter", "-", stdin=bad)
    assert r.returncode == 1 and "number of arguments to add must be positive" in r.stderr
    r = opt("--ascendc-no-such-stage", EXAMPLES / "broadcast_add_reduce.mlir")
    assert r.returncode == 1 and "Unknown command line argument" in r.stderr


def test_library_group_source_file_holds_its_descriptor_only(tmp_path):
    from ascend_mlir_b200.runtime.compiler import compile_kernel
    out = tmp_path / "step8_kernel.cpp"
    r = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cann", str(EXAMPLES / "matmul_add_leakyrelu.mlir"), "-o", str(out)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    text = out.read_text()
    assert "is a kernel of the runtime library" in text and 'extern "C"' not in text
    blob = compile_kernel(out, tmp_path / "artifact", "matmul_add_leakyrelu").read_bytes()
    assert int.from_bytes(blob[4:8], "little") == 1
    assert json.loads(blob[12:])["kernel_class"] == "matmul"


@pytest.mark.skipif(REFERENCE is None or not REFERENCE.exists(), reason="AFIR_REFERENCE_EXAMPLES does not name the reference's examples/")
@pytest.mark.parametrize("example", ["broadcast-add-reduce", "split-relu-brc-add-mul", "add-broadcast-concat",
                                     "relu-broadcast-transpose", "gather-elementwise-fusion", "matmul-add-leakyrelu"])
def test_reference_schedule_files_run_through_every_stage(tmp_path, example):
    """The reference's own step2_transform.mlir files (payload already fused, schedule beside it) through the stage
    sequence of its run.sh: same group as its step0_input.mlir gives."""
    scheduled = REFERENCE / example / "step2_transform.mlir"
    src = scheduled
    for i, flags in enumerate(REFERENCE_STAGES[2:], start=2):
        dst = tmp_path / f"stage{i}.mlir"
        r = opt(*flags, src, "-o", dst)
        assert r.returncode == 0, (flags, r.stderr)
        src = dst
    assert "afir.tile_index_args" in src.read_text() and "transform.named_sequence" not in src.read_text()
    got = translate(src)
    want = translate(REFERENCE / example / "step0_input.mlir")
    assert got["kernel_class"] == want["kernel_class"]
    assert body_of(got) == body_of(want) and got.get("matmul") == want.get("matmul")


# ---- fusion passes rewrite the IR -----------------------------------------------------------------------------------------
def count_generics(text):
    return sum(1 for line in text.splitlines() if "linalg.generic" in line and not line.strip().startswith("//"))


def test_fuse_elementwise_ops_leaves_one_generic_with_the_fused_body(tmp_path):
    """In the style of the reference's pass tests (test/Conversion/mark-structured-ops.mlir): the printed IR is checked."""
    src = EXAMPLES / "broadcast_add_reduce.mlir"
    assert count_generics(src.read_text()) == 2
    r = opt("--linalg-fuse-elementwise-ops", src)
    assert r.returncode == 0, r.stderr
    out = r.stdout
    assert count_generics(out) == 1
    assert 'iterator_types = ["parallel", "reduction"]' in out
    assert "ins(%b, %x : tensor<?xf32>, tensor<?x?xf32>) outs(%init : tensor<?xf32>)" in out
    # broadcast + add inlined into the reduction body: acc + (b[m] + x[m, n])
    assert "%f0 = arith.addf %in0, %in1 : f32" in out and "%sum = arith.addf %acc, %f0 : f32" in out
    assert 'afir.fused_group = "row_reduce"' in out
    # the rewritten module is the same group: it translates to the same descriptor
    fused = tmp_path / "fused.mlir"
    fused.write_text(out)
    a, b = translate(src), translate(fused)
    assert (a["kernel_class"], body_of(a), views_of(a)) == (b["kernel_class"], body_of(b), views_of(b))
    # running the pass again changes nothing more
    again = opt("--linalg-fuse-elementwise-ops", fused)
    assert again.returncode == 0 and count_generics(again.stdout) == 1


def test_fuse_elementwise_chain_with_constants_and_broadcasts(tmp_path):
    text = """#full = affine_map<(d0, d1) -> (d0, d1)>
#row = affine_map<(d0, d1) -> (d1)>
func.func @gated(%x: tensor<64x128xf16>, %s: tensor<128xf16>) -> tensor<64x128xf16> {
  %zero = arith.constant 0.0 : f16
  %e0 = tensor.empty() : tensor<64x128xf16>
  %a = linalg.generic {indexing_maps = [#full, #row, #full], iterator_types = ["parallel", "parallel"]}
      ins(%x, %s : tensor<64x128xf16>, tensor<128xf16>) outs(%e0 : tensor<64x128xf16>) {
  ^bb0(%xv: f16, %sv: f16, %o: f16):
    %m = arith.mulf %xv, %sv : f16
    linalg.yield %m : f16
  } -> tensor<64x128xf16>
  %e1 = tensor.empty() : tensor<64x128xf16>
  %b = linalg.generic {indexing_maps = [#full, #full], iterator_types = ["parallel", "parallel"]}
      ins(%a : tensor<64x128xf16>) outs(%e1 : tensor<64x128xf16>) {
  ^bb0(%av: f16, %o: f16):
    %r = arith.maximumf %av, %zero : f16
    %t = arith.addf %r, %av : f16
    linalg.yield %t : f16
  } -> tensor<64x128xf16>
  return %b : tensor<64x128xf16>
}
"""
    r = opt("--linalg-fuse-elementwise-ops", stdin=text)
    assert r.returncode == 0, r.stderr
    assert count_generics(r.stdout) == 1
    assert "%cst0 = arith.constant 0.000000e+00 : f16" in r.stdout
    assert "%f0 = arith.mulf %in0, %in1 : f16" in r.stdout and "%f1 = arith.maximumf %f0, %cst0 : f16" in r.stdout
    assert "%f2 = arith.addf %f1, %f0 : f16" in r.stdout and "linalg.yield %f2 : f16" in r.stdout
    plain, fused = tmp_path / "plain.mlir", tmp_path / "fused.mlir"
    plain.write_text(text)
    fused.write_text(r.stdout)
    a, b = translate(plain), translate(fused)
    assert (body_of(a), views_of(a)) == (body_of(b), views_of(b))


def test_groups_the_rewrite_does_not_cover_keep_their_ops():
    for name in ("split_relu_broadcast_add_mul", "matmul_add_leakyrelu"):
        src = EXAMPLES / f"{name}.mlir"
        r = opt("--linalg-fuse-elementwise-ops", src)
        assert r.returncode == 0, r.stderr
        assert count_generics(r.stdout) == count_generics(src.read_text())
        assert "afir.fused_group" in r.stdout


@pytest.mark.skipif(REFERENCE is None or not REFERENCE.exists(), reason="AFIR_REFERENCE_EXAMPLES does not name the reference's examples/")
def test_fuse_gather_elementwise_builds_the_reference_form(tmp_path):
    """relu -> index_select -> add of the reference's gather example (three generics) becomes the single gather generic
    its step2_transform.mlir holds: indices and bias as inputs, relu after the tensor.extract, gather_dim = 1."""
    src = REFERENCE / "gather-elementwise-fusion" / "step0_input.mlir"
    assert count_generics(src.read_text()) == 3
    r = opt("--mark-structured-ops", "--fuse-gather-elementwise", src)
    assert r.returncode == 0, r.stderr
    out = r.stdout
    assert count_generics(out) == 1 and "gather_dim = 1 : i64" in out
    assert "%pos = linalg.index 0 : index" in out and "tensor.extract %data[%pos, %picked]" in out
    assert "arith.maximumf %gathered, %cst0 : f16" in out
    fused = tmp_path / "fused.mlir"
    fused.write_text(out)
    a, b = translate(src), translate(fused)
    assert (a["kernel_class"], a["gather"], body_of(a)) == (b["kernel_class"], b["gather"], body_of(b))


@pytest.mark.skipif(REFERENCE is None or not REFERENCE.exists(), reason="AFIR_REFERENCE_EXAMPLES does not name the reference's examples/")
@pytest.mark.parametrize("example", ["add-broadcast-concat", "broadcast-add-reduce", "gather-elementwise-fusion",
                                     "relu-broadcast-transpose", "split-relu-brc-add-mul", "matmul-add-leakyrelu"])
def test_reference_example_scripts_drive_these_tools(tmp_path, example):
    """The reference's own examples/<name>/run.sh, copied beside a copy of its scripts/ directory and started with
    AFIR_OPT / AFIR_TRANSLATE / RUNTIME_SESSION naming this repository's tools: every compile stage passes (parse, fuse,
    schedule -- also preloaded from a transform library --, the lowering stages under the reference's names, codegen,
    data generation, runtime-session compile + plan) and the script arrives at its run stage, which needs a GPU.  The
    matmul example arrives at the point where it builds the reference's own mix-compiler from an LLVM tree, which
    has no counterpart here."""
    import shutil
    root = tmp_path / "checkout"
    shutil.copytree(REFERENCE / example, root / "examples" / example)
    if (REFERENCE.parent / "scripts").exists():
        shutil.copytree(REFERENCE.parent / "scripts", root / "scripts")
    for path in root.rglob("*"):
        path.chmod(path.stat().st_mode | 0o200)
    env = {**os.environ, "AFIR_OPT": str(BIN / "afir-opt"), "AFIR_TRANSLATE": str(BIN / "afir-translate"),
           "RUNTIME_SESSION": str(BIN / "runtime-session")}
    r = subprocess.run(["bash", "run.sh"], cwd=root / "examples" / example, env=env, capture_output=True, text=True, timeout=600)
    log = r.stdout + r.stderr
    assert "Unknown command line argument" not in log and "error: line" not in log, log[-2000:]
    if example == "matmul-add-leakyrelu":
        assert "[STAGE 8] Codegen" in log and "Bootstrap RuntimeMix tools" in log and r.returncode == 2, log[-2000:]
        assert (root / "examples" / example / "step8_kernel.cpp").read_text().startswith("// afir-cuda-launch-descriptor-begin")
        return
    assert "[STAGE 10]" in log and "session.plan[0]=main" in log, log[-2000:]
    # at the run stage (some scripts keep the tool's output in a file of their own): validated on a machine with a GPU,
    # stopped at the device on one without; never at the bindings
    after = log[log.index("[STAGE 10]"):]
    for kept in (root / "examples" / example).rglob("runtime_session*.log"):
        after += kept.read_text()
    assert "session.backend=sim" in after  # the line the scripts grep for
    assert "session.validation=pass" in after or "session.error_stage=device" in after, after[-2000:]
    assert r.returncode == (0 if "session.validation=pass" in after else r.returncode)
