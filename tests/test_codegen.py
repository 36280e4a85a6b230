"""The kernel generator and its compile step, without a GPU.

`afir-translate -mlir-to-cuda-kernel` prints the CUDA source of a fused group's kernel and `afirt_compiler_compile`
compiles it for sm_100a with NVRTC.  The text checks follow the style of the reference's emitter tests
(test/Target/cann-translate.mlir, test/Conversion/canonicalize-cann-signature.mlir): the kernel signature
(inputs..., outputs..., workspace, TilingData), the all-int64 TilingData struct with tile parameters first and
dim_arg<N>_<D> after them, and the fused body as one call per arith op.
"""
import copy
import json
import re
import subprocess
from pathlib import Path

import pytest

from ascend_mlir_b200 import build as lib_build
from ascend_mlir_b200 import descriptors
from ascend_mlir_b200.runtime.compiler import compile_kernel

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "ascend_mlir_b200" / "bin"
EXAMPLES = ROOT / "ascend_mlir_b200" / "examples"


@pytest.fixture(scope="module", autouse=True)
def built():
    lib_build.build()


def kernel_source(mlir, *extra):
    return subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda-kernel", str(mlir), *map(str, extra)],
                          capture_output=True, text=True)


def compiled(tmp_path, spec, descriptor=None):
    """Runs afirt_compiler_compile on a descriptor and returns (json, cubin, source) of the container."""
    d = descriptor or spec.descriptor
    src = tmp_path / f"{d['kernel']}.cuda.json"
    src.write_text(json.dumps(d))
    blob = compile_kernel(src, tmp_path / f"out_{d['kernel']}", d["kernel"]).read_bytes()
    assert blob[:4] == b"AFCU"
    version, json_len = int.from_bytes(blob[4:8], "little"), int.from_bytes(blob[8:12], "little")
    if version == 1:
        return blob[12:12 + json_len], b"", ""
    off = 12 + json_len
    n = int.from_bytes(blob[off:off + 4], "little")
    cubin = blob[off + 4:off + 4 + n]
    off += 4 + n
    m = int.from_bytes(blob[off:off + 4], "little")
    return blob[12:12 + json_len], cubin, blob[off + 4:off + 4 + m].decode()


def test_elementwise_chain_source_has_the_reference_signature_and_a_straight_line_body():
    r = kernel_source(EXAMPLES / "elementwise_chain.mlir")
    assert r.returncode == 0, r.stderr
    src = r.stdout
    assert 'extern "C" __global__ void __launch_bounds__(512) elementwise_chain(const void *arg0, const void *arg1, void *arg2, ' \
           "void *workspace, const __grid_constant__ TilingData t)" in src
    # out = (a + b) * b: one call per op, each rounding to the element type (the packs use __fadd_rn / __fmul_rn)
    assert "const P r0 = P::add(v[0], v[1]);" in src and "const P r1 = P::mul(r0, v[1]);" in src and "return r1;" in src
    assert "PackF32" in src and "PackF16" not in src
    # static shapes fold: both operands and the output are walked contiguously, so the three dims collapse to one
    assert "const long long d0 = 1LL, d1 = 1LL, d2 = 4096LL * rows0;" in src


def test_tiling_data_is_all_int64_tile_parameters_first_then_dims_then_the_runtime_words():
    spec = descriptors.split_relu_bias_mul()
    out = subprocess.run([str(BIN / "afir-translate"), "-mlir-to-cuda-kernel", str(EXAMPLES / "split_relu_broadcast_add_mul.mlir")],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    struct = out.stdout[out.stdout.index("struct TilingData {"):out.stdout.index("};", out.stdout.index("struct TilingData {"))]
    fields = re.findall(r"long long ([A-Za-z_0-9, ]+);", struct)
    names = [n.strip() for f in fields for n in f.split(",")]
    assert names[-8:] == ["afir_row_begin", "afir_row_end", "afir_p0", "afir_p1", "afir_p2", "afir_p3", "afir_p4", "afir_p5"]
    assert names[:2] == ["CTA_THREADS", "UNROLL"]
    assert spec.descriptor["tiling"][0]["name"] == "CTA_THREADS"
    # relu, + bias, * h1, with the constant spelled by its bits
    assert "P::max(v[0], P::constant(__uint_as_float(0x00000000u)))" in out.stdout
    # the two halves of x are two views of argument 0, the second one 1024 elements in
    assert out.stdout.count("static_cast<const char *>(arg0)") == 2 and "(1024LL) * (1LL)" in out.stdout


def test_dynamic_dims_are_read_from_tiling_data(tmp_path):
    _, cubin, src = compiled(tmp_path, descriptors.add_mul())
    assert cubin[:4] == b"\x7fELF"
    assert "long long dim_arg0_0;" in src and "long long dim_arg0_1;" in src
    assert "t.dim_arg0_1" in src and ": t.dim_arg0_0;" in src  # rows0 falls back to the leading dim without a row window


def test_row_reduction_has_three_entries(tmp_path):
    spec = descriptors.bcast_add_rowsum("f32")
    _, cubin, src = compiled(tmp_path, spec)
    assert cubin[:4] == b"\x7fELF"
    for entry in (f"{spec.name}(", f"{spec.name}__staged(", f"{spec.name}__finalize("):
        assert re.search(r'extern "C" __global__ void .*' + re.escape(entry), src), entry
    assert "rowReduceTeams<PackF32, FusedBody0, true>" in src and "rowReduceStream<PackF32, FusedBody0>" in src
    assert "sp.streamViewIndex = 1;" in src  # b[m, n] is the streamed view, a[m] the broadcast one


def test_which_generated_kernels_wait_for_their_grid_dependencies(tmp_path):
    """Elementwise and row-reduction kernels begin with gridDependencyPrologue() and their module says so with a marker
    kernel (the runtime then launches them with programmatic stream serialisation); gather kernels, one short CTA per
    tile, have neither."""
    marker = "void afir_waits_for_grid_dependencies() {}"
    _, _, src = compiled(tmp_path, descriptors.bcast_add_rowsum("f32"))
    assert marker in src and src.count("gridDependencyPrologue();") == 3  # main, staged, finalize
    _, _, src = compiled(tmp_path, descriptors.add_mul())
    assert marker in src and src.count("gridDependencyPrologue();") == 1
    _, cubin, src = compiled(tmp_path, descriptors.gather_rows_scale_resid())
    assert cubin[:4] == b"\x7fELF" and marker not in src and "gridDependencyPrologue" not in src


def test_sixteen_bit_groups_compile_with_their_packs(tmp_path):
    for spec in (descriptors.split_relu_bias_mul(), descriptors.gather_rows_scale_resid(), descriptors.bcast_add_rowsum("f16")):
        _, cubin, src = compiled(tmp_path, spec)
        assert cubin[:4] == b"\x7fELF", spec.name
        assert ("PackF16" in src) != ("PackBF16" in src)


def test_integer_constants_are_emitted_exactly(tmp_path):
    d = copy.deepcopy(descriptors.add_mul("i32", name="int_chain").descriptor)
    d["body"] = [descriptors.op("addi", "v0", 16777217), descriptors.op("muli", "%0", "v1"), descriptors.op("subi", "%1", -2147483647)]
    _, cubin, src = compiled(tmp_path, None, d)
    assert cubin[:4] == b"\x7fELF"
    assert "P::constantInt(16777217)" in src and "P::constantInt(-2147483647)" in src  # 2^24 + 1 survives


def test_groups_of_the_library_get_no_generated_source(tmp_path):
    r = kernel_source(EXAMPLES / "matmul_add_leakyrelu.mlir")
    assert r.returncode == 1 and "hand-written tcgen05 kernel" in r.stderr
    r = kernel_source(EXAMPLES / "transpose_2d.mlir")
    assert r.returncode == 1 and "no kernel source is generated" in r.stderr
    # a bare permutation written as an elementwise group (a copy through a transposed view) stays with the library's
    # transpose kernels: the compile step succeeds, descriptor only
    d = copy.deepcopy(descriptors.transposed_add_mul("f16").descriptor)
    d["kernel"] = "transposed_copy"
    d["num_inputs"] = 1
    d["loads"] = d["loads"][:1]
    d["store"]["arg"] = 1
    d["body"] = []
    _, cubin, src = compiled(tmp_path, None, d)
    assert cubin == b"" and src == ""


def test_transposed_operand_gets_the_register_block_loop(tmp_path):
    """A group that reads an operand through a transposed view: its kernel holds the register-block loop (16-byte pieces
    on every side, transposed in registers) beside the element-wise one and picks at run time; CTAs of 256 threads."""
    r = kernel_source(EXAMPLES / "transposed_add.mlir")
    assert r.returncode == 0, r.stderr
    assert "elementwiseBlocksTiles<" in r.stdout and "kViewTransposed" in r.stdout and "__launch_bounds__(256, 3)" in r.stdout
    for dtype in ("f16", "f32"):
        _, cubin, src = compiled(tmp_path, descriptors.transposed_add_mul(dtype))
        assert cubin[:4] == b"\x7fELF"
        assert '#include "kernels/elementwise_blocks_skel.cuh"' in src
        assert "bp.kind[0] = kViewTransposed" in src and "bp.kind[1] = kViewRowMajor" in src and "bp.kind[2] = kViewInnerBroadcast" in src
        assert "elementwiseTiles<" in src  # the element-wise fallback for unaligned operands
        assert "void afir_ctas_of_256_threads() {}" in src  # the runtime launches 256 threads whatever the tiling says


def test_register_block_kernels_are_compiled_for_three_ctas_per_sm_where_the_blocks_fit(tmp_path):
    """(a^T + b) * c keeps two views of 8 x 8 blocks in registers (c is one element per row): three CTAs per SM.  With
    three row-major operands beside the transposed one, 16-bit blocks no longer fit in 80 registers: two CTAs per SM."""
    _, _, src = compiled(tmp_path, descriptors.transposed_add_mul("f16"))
    assert "__launch_bounds__(256, 3)" in src
    dims = [("dim_arg0_0", "M"), ("dim_arg0_1", "N")]
    dom = ["dim_arg0_1", "dim_arg0_0"]
    loads = [{"arg": 0, "shape": ["dim_arg0_0", "dim_arg0_1"], "map": [1, 0]}] + [{"arg": i, "shape": dom, "map": [0, 1]} for i in (1, 2, 3)]
    body = {"domain": dom, "loads": loads, "store": {"arg": 4, "shape": dom, "map": [0, 1]},
            "body": [descriptors.op("addf", "v0", "v1"), descriptors.op("addf", "%0", "v2"), descriptors.op("mulf", "%1", "v3")]}
    for dtype, bounds in (("f16", "__launch_bounds__(256) "), ("f32", "__launch_bounds__(256, 3) ")):
        wide = descriptors._spec("four_operands", "elementwise", dtype, 4, 1, descriptors._EW_TILE, dims, body, descriptors._EW_LAUNCH)
        _, cubin, src = compiled(tmp_path, wide)
        assert cubin[:4] == b"\x7fELF" and bounds + "four_operands(" in src


@pytest.mark.parametrize("example", ["elementwise_chain", "split_relu_broadcast_add_mul", "broadcast_add_reduce",
                                     "gather_elementwise", "integer_chain"])
def test_every_generated_example_compiles_to_a_cubin(tmp_path, example):
    cubin = tmp_path / f"{example}.cubin"
    r = kernel_source(EXAMPLES / f"{example}.mlir", "-o", tmp_path / f"{example}.cu", "--cubin-out", cubin)
    assert r.returncode == 0, r.stderr
    assert cubin.read_bytes()[:4] == b"\x7fELF"
    assert (tmp_path / f"{example}.cu").read_text().startswith('#include "kernels/')


def test_multi_group_descriptor_is_one_kernel(tmp_path):
    """Split rows / concat: two groups writing the two halves of one output become two blocks of one kernel."""
    _, cubin, src = compiled(tmp_path, descriptors.split_rows_relu_bias_scale())
    assert cubin[:4] == b"\x7fELF"
    # one kernel for all groups, beside the empty marker kernel that says "these kernels wait for their grid dependencies"
    assert src.count('extern "C" __global__') == 2 and 'void afir_waits_for_grid_dependencies() {}' in src
    assert src.count("gridDependencyPrologue();") == 1
    assert "// group 0" in src and "// group 1" in src and "FusedBody1" in src
    # the second half starts dim_arg1_0 rows into argument 0 and argument 5
    assert "(t.dim_arg1_0) * (t.dim_arg0_1)" in src


def test_source_that_does_not_compile_fails_the_compile_step(tmp_path):
    d = copy.deepcopy(descriptors.add_mul().descriptor)
    d["tiling"].append({"name": "dim arg", "type": "int64"})   # sanitised to an identifier, still compiles
    d["tiling"].append({"name": "dim_arg", "type": "int64"})   # ... but collides with this one: no source, library kernels
    src = tmp_path / "add_mul.cuda.json"
    src.write_text(json.dumps(d))
    out = compile_kernel(src, tmp_path / "out", "add_mul")
    manifest = dict(line.split("=", 1) for line in (tmp_path / "out" / "manifest.txt").read_text().splitlines())
    assert manifest["codegen"].startswith("library (two tiling fields map to one identifier")
    assert int.from_bytes(out.read_bytes()[4:8], "little") == 1
