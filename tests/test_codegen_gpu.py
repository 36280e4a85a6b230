"""Generated kernels on the GPU: what the kernel generator emits for a fused group, compiled with NVRTC, loaded
with cuModuleLoadData and launched with cuLaunchKernel as <kernel>(inputs..., outputs..., workspace, TilingData),
must give the same bits as the library's prebuilt kernels and as the CPU oracle.

Three layers: (1) dedicated cases that check which code ran (afirt_executor_last_launch_generated) -- chains no
prebuilt body matches, integer constants beyond 2^24, every row-reduction plan, gathers, split/concat descriptors,
artifacts compiled ahead of time; (2) the whole parity suite once more with AFIR_CUDA_CODEGEN=always, so every
shape, ragged edge and error path the prebuilt kernels are tested on also runs on generated code wherever a
generated kernel exists; (3) the four bandwidth-bound configurations at full size (row windows of the pipelined
host path included).
"""
import copy
import json

import numpy as np
import pytest

import test_parity_gpu as parity
from test_parity_gpu import rt  # noqa: F401  (module-scoped runtime fixture)

from ascend_mlir_b200 import configs, descriptors
from ascend_mlir_b200.runtime.compiler import compile_kernel
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def generated_everywhere(monkeypatch):
    monkeypatch.setenv("AFIR_CUDA_CODEGEN", "always")


def variant(spec, name, body, dtype=None):
    d = copy.deepcopy(spec.descriptor)
    d["kernel"] = name
    d["body"] = body
    if dtype:
        d["dtype"] = dtype
    return d


def run_descriptor(rt, d, spec, inputs, out, shape, **tile):
    rt.run(descriptors.container(d), d["kernel"], inputs, [out], spec.pack(shape, **tile))
    return out


# ---- (1) which code ran, and that it is right -----------------------------------------------------------------------
@pytest.mark.parametrize("M,N", [(33, 64), (257, 1023), (1, 1), (512, 4096)])
def test_unmatched_chain_runs_generated_code_in_the_default_mode(rt, monkeypatch, M, N):
    monkeypatch.delenv("AFIR_CUDA_CODEGEN")  # the default, "auto": generated code where the library would interpret
    spec = descriptors.add_mul()
    d = variant(spec, "sub_div_min", [descriptors.op("subf", "v0", "v1"), descriptors.op("divf", "%0", "v1"),
                                      descriptors.op("minimumf", "%1", "v0")])
    rng = np.random.default_rng(8)
    a = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    b = rng.uniform(0.5, 1.5, (M, N)).astype(np.float32)
    out = run_descriptor(rt, d, spec, [a, b], np.zeros_like(a), {"M": M, "N": N})
    assert rt.last_launch_generated and rt.last_launch_count >= 1  # (one launch per row chunk of the pipelined host path)
    assert np.array_equal(out, np.minimum((a - b) / b, a))
    # the same group on the library's interpreter: same bits
    monkeypatch.setenv("AFIR_CUDA_CODEGEN", "never")
    again = run_descriptor(rt, d, spec, [a, b], np.zeros_like(a), {"M": M, "N": N})
    assert not rt.last_launch_generated
    assert again.tobytes() == out.tobytes()
    # the default mode: elementwise, row-reduction and row-gather groups run generated code; matmul and transposes
    # are the library's kernels
    monkeypatch.delenv("AFIR_CUDA_CODEGEN")
    w = configs.elementwise_chain(64, 256, seed=1)
    rt.run(w.spec.binary, w.spec.name, w.inputs, [w.new_output()], w.tiling())
    assert rt.last_launch_generated
    w = configs.broadcast_add_reduce(64, 256, seed=1)
    rt.run(w.spec.binary, w.spec.name, w.inputs, [w.new_output()], w.tiling())
    assert rt.last_launch_generated
    w = configs.gather_elementwise(512, 64, 128, seed=1)
    rt.run(w.spec.binary, w.spec.name, w.inputs, [w.new_output()], w.tiling())
    assert rt.last_launch_generated
    w = configs.matmul_add_leakyrelu(128, 256, 64, seed=1)
    rt.run(w.spec.binary, w.spec.name, w.inputs, [w.new_output()], w.tiling(), magic=w.spec.magic)
    assert not rt.last_launch_generated


def test_six_op_chain_bit_exact_f32_and_f16(rt):
    body = [descriptors.op("mulf", "v0", "v1"), descriptors.op("addf", "%0", "v0"), descriptors.op("maximumf", "%1", 0.25),
            descriptors.op("subf", "%2", "v1"), descriptors.op("mulf", "%3", "%0"), descriptors.op("minimumf", "%4", 1.5)]
    for dtype, np_t in (("f32", np.float32), ("f16", np.float16)):
        spec = descriptors.add_mul(dtype)
        d = variant(spec, "six_ops", body)
        rng = np.random.default_rng(81)
        a = rng.uniform(-2, 2, (300, 520)).astype(np_t)
        b = rng.uniform(-2, 2, (300, 520)).astype(np_t)
        out = run_descriptor(rt, d, spec, [a, b], np.zeros_like(a), {"M": 300, "N": 520})
        assert rt.last_launch_generated
        r0 = (a * b).astype(np_t)
        r1 = (r0 + a).astype(np_t)
        r2 = np.maximum(r1, np_t(0.25))
        r3 = (r2 - b).astype(np_t)
        r4 = (r3 * r0).astype(np_t)
        want = np.minimum(r4, np_t(1.5))
        assert out.tobytes() == want.tobytes()


def test_integer_constants_beyond_2_pow_24_are_exact(rt, monkeypatch):
    spec = descriptors.add_mul("i32", name="int_chain")
    body = [descriptors.op("addi", "v0", 16777217), descriptors.op("muli", "%0", "v1"), descriptors.op("subi", "%1", -2147483647)]
    d = variant(spec, "int_chain", body)
    rng = np.random.default_rng(82)
    a = rng.integers(-2 ** 31, 2 ** 31, (65, 128), dtype=np.int64).astype(np.int32)
    b = rng.integers(-2 ** 31, 2 ** 31, (65, 128), dtype=np.int64).astype(np.int32)
    want = (((a.astype(np.int64) + 16777217) * b.astype(np.int64) + 2147483647) & 0xFFFFFFFF).astype(np.uint32).view(np.int32)
    for mode in ("always", "never"):  # generated code and the library's interpreter read the same exact constant
        monkeypatch.setenv("AFIR_CUDA_CODEGEN", mode)
        out = run_descriptor(rt, d, spec, [a, b], np.zeros_like(a), {"M": 65, "N": 128})
        assert rt.last_launch_generated == (mode == "always")
        assert np.array_equal(out, want), mode


@pytest.mark.parametrize("M,N,split,launches", [(5, 40000, 4, 2), (300, 1000, 0, 1), (1500, 8192, 0, 1), (7, 33, 0, 1), (2000, 4096, 0, 1)])
def test_row_reduction_plans_on_generated_code(rt, monkeypatch, M, N, split, launches):
    """Teams with plain loads, column slices through the workspace + finalize, and the bulk-copy staged loop
    (1500 x 8192 f32 and 2000 x 4096: at least 148 x 8 rows of 16 KB or more), each with a body the library has no kernel for."""
    monkeypatch.setenv("AFIR_CUDA_NO_PIPELINE", "1")  # one launch for the whole problem, not one per row chunk of the host path
    spec = descriptors.bcast_add_rowsum("f32")
    d = variant(spec, "sub_mul_rowsum", [descriptors.op("subf", "v1", "v0"), descriptors.op("mulf", "%0", "v1")])
    rng = np.random.default_rng(83)
    a = rng.uniform(-1, 1, M).astype(np.float32)
    x = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    tile = {"SPLIT_N": split} if split else {}
    out = run_descriptor(rt, d, spec, [a, x], np.zeros(M, np.float32), {"M": M, "N": N}, **tile)
    assert rt.last_launch_generated and rt.last_launch_count == launches
    terms = ((x - a[:, None]).astype(np.float32) * x).astype(np.float32).astype(np.float64)
    assert np.all(np.abs(out - terms.sum(axis=1)) <= 1e-5 * np.abs(terms).sum(axis=1) + 1e-30)


def test_generated_and_prebuilt_reductions_agree_bit_for_bit(rt, monkeypatch):
    """Same loop templates, same launch plan, same summation order: identical bits, plan by plan."""
    for M, N, tile in ((5, 40000, {"SPLIT_N": 4}), (300, 1000, {}), (1500, 8192, {})):
        w = configs.broadcast_add_reduce(M, N, seed=84)
        outs = {}
        for mode in ("always", "never"):
            monkeypatch.setenv("AFIR_CUDA_CODEGEN", mode)
            out = w.new_output()
            rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling(**tile))
            assert rt.last_launch_generated == (mode == "always")
            outs[mode] = out
        assert outs["always"].tobytes() == outs["never"].tobytes(), (M, N)


@pytest.mark.parametrize("T,W,R", [(4096, 256, 2048), (50, 7, 20), (65536, 64, 5000)])
def test_gather_with_an_unmatched_body_runs_generated_code(rt, T, W, R):
    w = configs.gather_elementwise(T, W, R, seed=85)
    # (table[idx] + resid) * scale instead of the benchmark's table[idx] * scale + resid
    d = variant(w.spec, "gather_add_mul", [descriptors.op("addf", "v0", "v2"), descriptors.op("mulf", "%0", "v1")])
    out = w.new_output()
    rt.run(descriptors.container(d), "gather_add_mul", w.inputs, [out], w.tiling())
    assert rt.last_launch_generated
    table, idx, scale, resid = w.inputs
    g = oracle.bf16_to_f32(table)[idx]
    s1 = oracle.f32_to_bf16(g + oracle.bf16_to_f32(resid))
    want = oracle.f32_to_bf16(oracle.bf16_to_f32(s1) * oracle.bf16_to_f32(scale)[None, :])
    assert np.array_equal(out, want)


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("M,N", [(512, 256), (520, 264), (1000, 24), (24, 1000), (3, 5), (257, 129), (1, 4096), (4096, 1), (1, 1)])
def test_transposed_operand_with_an_unmatched_body_runs_the_generated_block_loop(rt, dtype, M, N):
    """out[n, m] = min(a[m, n] - b[n, m], c[n]): no body of the library matches, so before generated code covered
    transposed operands this ran op by op; whole blocks, ragged blocks and shapes whose strides rule 16-byte pieces out
    (the kernel's element-wise loop), and extents of one (where the runtime's view of the collapsed domain has no transposed
    operand left, while the kernel is still the 256-thread one), against numpy with rounding after every op."""
    rng = np.random.default_rng(91)
    a = rng.standard_normal((M, N)).astype(dtype)
    b = rng.standard_normal((N, M)).astype(dtype)
    c = rng.standard_normal(N).astype(dtype)
    spec = descriptors.transposed_add_mul("f16" if dtype == np.float16 else "f32")
    d = variant(spec, "transposed_sub_min", [descriptors.op("subf", "v0", "v1"), descriptors.op("minimumf", "%0", "v2")])
    out = run_descriptor(rt, d, spec, [a, b, c], np.zeros((N, M), dtype), {"M": M, "N": N})
    assert rt.last_launch_generated
    want = np.minimum((a.T - b).astype(dtype), c[:, None]).astype(dtype)
    assert out.tobytes() == want.tobytes()


@pytest.mark.parametrize("unroll", [1, 2])
@pytest.mark.parametrize("threads,block_dim", [(128, 0), (256, 0), (512, 5), (128, 100000)])
def test_generated_gather_entries_and_grids(rt, unroll, threads, block_dim):
    """Both entries of a generated row gather (one or two vectors per thread in flight), with the default bounded grid
    (more tiles than CTAs: every CTA walks several), a grid of five CTAs and one asked for above the tile count; 300 000
    rows of 24 columns (48-byte rows: 16-byte vectors, three per row) and an unaligned width (element access)."""
    for T, W, R in ((70000, 24, 300000), (3000, 7, 9001)):
        w = configs.gather_elementwise(T, W, R, seed=87)
        out = w.new_output()
        rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling(UNROLL=unroll, CTA_THREADS=threads), block_dim=block_dim)
        assert rt.last_launch_generated
        assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs)), (T, W, R)


def test_gather_out_of_range_indices_are_counted_by_generated_code(rt):
    from ascend_mlir_b200.runtime import ExecutorError
    w = configs.gather_elementwise(100, 16, 40, seed=13)
    w.inputs[1][7] = 100
    w.inputs[1][9] = -1
    out = np.full(w.out_shape, 0x7FC0, np.uint16)
    with pytest.raises(ExecutorError, match=r"gather index out of range \(2 indices\)"):
        rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling())
    assert rt.last_launch_generated
    w.inputs[1][[7, 9]] = 0  # the context survives and the next call works
    rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling())
    assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs))


def test_split_rows_concat_descriptor_is_one_generated_launch(rt, golden_dir):
    g = dict(np.load(golden_dir / "split_relu_brc_add_mul.npz"))
    spec = descriptors.split_rows_relu_bias_scale()
    inputs = [g["input_a"], g["bias0"], g["bias1"], g["scale0"], g["scale1"]]
    M, N = inputs[0].shape
    out = np.zeros((M, N), np.float16)
    rt.run(spec.binary, spec.name, inputs, [out], spec.pack({"M": M, "N": N, "HM": M // 2}))
    assert rt.last_launch_generated and rt.last_launch_count == 1  # two groups, one kernel
    want = oracle.split_rows_relu_bias_scale_f16(*inputs)
    assert out.tobytes() == want.tobytes()


def test_artifact_compiled_ahead_of_time_brings_its_device_binary(rt, tmp_path):
    """afirt_compiler_compile puts the cubin in the container; the executor loads it (no compile at run time)."""
    spec = descriptors.add_mul()
    d = variant(spec, "sub_div_min", [descriptors.op("subf", "v0", "v1"), descriptors.op("divf", "%0", "v1"),
                                      descriptors.op("minimumf", "%1", "v0")])
    src = tmp_path / "sub_div_min.cuda.json"
    src.write_text(json.dumps(d))
    blob = compile_kernel(src, tmp_path / "out", "sub_div_min").read_bytes()
    assert int.from_bytes(blob[4:8], "little") == 2
    rng = np.random.default_rng(86)
    a = rng.uniform(-1, 1, (129, 384)).astype(np.float32)
    b = rng.uniform(0.5, 1.5, (129, 384)).astype(np.float32)
    out = np.zeros_like(a)
    rt.run(blob, "sub_div_min", [a, b], [out], spec.pack({"M": 129, "N": 384}))
    assert rt.last_launch_generated
    assert np.array_equal(out, np.minimum((a - b) / b, a))


def test_tile_parameters_the_generated_loop_does_not_take_stay_on_the_library(rt):
    w = configs.elementwise_chain(513, 1024, seed=4)
    for unroll, generated in ((2, True), (4, False), (1, False)):
        out = w.new_output()
        rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling(UNROLL=unroll, CTA_THREADS=256), block_dim=7)
        assert rt.last_launch_generated == generated
        assert np.array_equal(out, oracle.add_mul_f32(*w.inputs))


# ---- (2) the parity suite again, on generated code wherever it exists ------------------------------------------------------
for _name in dir(parity):
    if _name.startswith("test_"):
        globals()[_name + "_generated"] = getattr(parity, _name)


# ---- (3) full-size configurations on generated code -------------------------------------------------------------------------
def test_full_size_configs_1_to_4_on_generated_code(rt):
    w = configs.elementwise_chain()
    out = w.new_output()
    rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling())
    assert rt.last_launch_generated
    assert np.array_equal(out, oracle.add_mul_f32(*w.inputs))

    w = configs.split_relu_broadcast_add_mul()
    out = w.new_output()
    rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling())
    assert rt.last_launch_generated
    assert np.array_equal(out.view(np.uint16), oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], 1).view(np.uint16))

    w = configs.broadcast_add_reduce()
    out = w.new_output()
    rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling())
    assert rt.last_launch_generated
    _, s64, abs64 = oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1], with_bounds=True)
    assert np.all(np.abs(out - s64) <= 1e-5 * abs64)

    w = configs.gather_elementwise()
    out = w.new_output()
    rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling())
    assert rt.last_launch_generated
    assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs))
