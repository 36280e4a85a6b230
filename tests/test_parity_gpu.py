"""GPU parity: every fused-group kernel, called through the afirt_* C-ABI, against the CPU oracle on the
same seeded inputs, plus the reference's own golden fixtures.  Bars: bit-exact for f32 elementwise,
for f16/bf16 chains (per-op rounding on both sides) and for all indexing; reductions within
1e-5 * sum|x| per row."""
import copy

import numpy as np
import pytest

from ascend_mlir_b200 import configs, descriptors
from ascend_mlir_b200.runtime import ExecutorError
from ascend_mlir_b200.runtime.executor import CudaRuntime
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    r = CudaRuntime()
    r.set_device(0)
    return r


def run(rt, spec, inputs, out, shape, block_dim=0, **tile):
    rt.run(spec.binary, spec.name, inputs, [out], spec.pack(shape, **tile), block_dim=block_dim, magic=spec.magic)
    assert rt.last_launch_count >= 1
    return out


def bits(x):
    return np.ascontiguousarray(x).view(np.uint16) if x.dtype == np.float16 else x


# ---- elementwise chain ----------------------------------------------------------------------------
@pytest.mark.parametrize("M,N", [(4096, 512), (1, 4), (3, 5), (257, 1023), (64, 4096), (1, 1)])
def test_add_mul_f32_bit_exact(rt, M, N):
    w = configs.elementwise_chain(M, N, seed=3)
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape)
    assert np.array_equal(out.view(np.uint32), oracle.add_mul_f32(*w.inputs).view(np.uint32))


@pytest.mark.parametrize("threads,unroll,block_dim", [(128, 1, 0), (256, 2, 7), (512, 4, 148), (256, 4, 1)])
def test_add_mul_tile_params_do_not_change_results(rt, threads, unroll, block_dim):
    w = configs.elementwise_chain(513, 1024, seed=4)
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape, block_dim=block_dim, CTA_THREADS=threads, UNROLL=unroll)
    assert np.array_equal(out, oracle.add_mul_f32(*w.inputs))


def test_add_mul_empty(rt):
    w = configs.elementwise_chain(0, 16)
    out = run_empty = np.zeros((0, 16), np.float32)
    rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling())
    assert run_empty.size == 0


def test_add_mul_special_values(rt):
    a = np.array([[np.nan, np.inf, -np.inf, -0.0, 1e-45, 3.4e38, 1.0, -1.0]], np.float32)
    b = np.array([[1.0, -np.inf, 2.0, 0.0, 1e-45, 3.4e38, np.nan, 1e-30]], np.float32)
    spec = descriptors.add_mul()
    out = run(rt, spec, [a, b], np.zeros_like(a), {"M": 1, "N": 8})
    want = oracle.add_mul_f32(a, b)
    assert np.array_equal(np.isnan(out), np.isnan(want))
    m = ~np.isnan(want)
    assert np.array_equal(out.view(np.uint32)[m], want.view(np.uint32)[m])


# ---- split / broadcast ------------------------------------------------------------------------------
@pytest.mark.parametrize("B,R,C,axis", [(4, 64, 256, 1), (4, 64, 256, 2), (2, 3, 8, 1), (3, 5, 7, 1), (1, 17, 24, 2)])
def test_split_relu_bias_mul_f16_bit_exact(rt, B, R, C, axis):
    w = configs.split_relu_broadcast_add_mul(B, R, C, bias_axis=axis, seed=5)
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape)
    want = oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], bias_axis=axis)
    assert np.array_equal(bits(out), bits(want))


def test_split_relu_negative_zero_and_nan(rt):
    x = np.zeros((1, 2, 16), np.float16)
    x[0, 0, :8] = [-0.0, 0.0, -1.0, np.nan, 6e-8, -6e-8, 65504, -65504]
    x[0, :, 8:] = 1.0
    bias = np.array([-0.0, 0.0], np.float16)
    spec = descriptors.split_relu_bias_mul(1)
    shape = {"B": 1, "R": 2, "C2": 16, "C": 8, "BIAS": 2}
    out = run(rt, spec, [x, bias], np.zeros((1, 2, 8), np.float16), shape)
    want = oracle.split_relu_bias_mul_f16(x, bias, 1)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(out), nan)
    assert np.array_equal(bits(out)[~nan], bits(want)[~nan])


def test_reference_split_example_golden(rt, golden_dir):
    g = dict(np.load(golden_dir / "split_relu_brc_add_mul.npz"))
    spec = descriptors.split_rows_relu_bias_scale()
    M, N = g["input_a"].shape
    out = run(rt, spec, [g["input_a"], g["bias0"], g["bias1"], g["scale0"], g["scale1"]], np.zeros((M, N), np.float16),
              {"M": M, "N": N, "HM": M // 2})
    # two halves, written in place of the concat: two launches of the library's kernel, or the two groups as one generated kernel
    assert rt.last_launch_count == (1 if rt.last_launch_generated else 2)
    want = oracle.split_rows_relu_bias_scale_f16(g["input_a"], g["bias0"], g["bias1"], g["scale0"], g["scale1"])
    assert np.array_equal(bits(out), bits(want))
    fails, _, _ = oracle.compare(out.astype(np.float32), g["output"].astype(np.float32), 1e-2, 1e-2)
    assert fails == 0


def test_reference_concat_example_golden(rt, golden_dir):
    g = dict(np.load(golden_dir / "add_broadcast_concat.npz"))
    spec = descriptors.add_mul_concat()
    M, N = g["input_b"].shape
    out = run(rt, spec, [g["input_a"], g["input_b"], g["input_c"], g["input_d"]], np.zeros((2 * M, N), np.float16),
              {"M": M, "N": N, "M2": 2 * M})
    assert np.array_equal(bits(out), bits(g["output"]))


def test_reference_transpose_example_golden_memcmp(rt, golden_dir):
    g = dict(np.load(golden_dir / "relu_broadcast_transpose.npz"))
    spec = descriptors.relu_bcast_transpose_add()
    N, M = g["input_data1"].shape
    out = run(rt, spec, [g["input_data0"], g["input_data1"]], np.zeros((N, M), np.float16), {"M": M, "N": N})
    assert out.tobytes() == g["output_expected"].tobytes()


@pytest.mark.parametrize("R,C,dtype", [(640, 500, np.float16), (65, 129, np.float32), (1, 7, np.float16), (2048, 1024, np.float32)])
def test_transpose_2d(rt, R, C, dtype):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((R, C)).astype(dtype)
    spec = descriptors.transpose_2d("f16" if dtype == np.float16 else "f32")
    out = run(rt, spec, [x], np.zeros((C, R), dtype), {"R": R, "C": C})
    assert out.tobytes() == oracle.transpose_2d(x).tobytes()


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("warp_rows", [1, 2, 4, 8])
def test_transpose_2d_every_warp_arrangement(rt, dtype, warp_rows):
    """Aligned operands take the register-block kernel: whole tiles, ragged tiles in both directions, and a
    shape smaller than one block, for every arrangement of the CTA's warps and for the tile kernel."""
    rng = np.random.default_rng(11)
    spec = descriptors.transpose_2d("f16" if dtype == np.float16 else "f32")
    for R, C in [(512, 256), (520, 264), (8, 8), (1000, 24), (24, 1000), (4, 4)]:
        x = rng.standard_normal((R, C)).astype(dtype)
        want = oracle.transpose_2d(x).tobytes()
        out = run(rt, spec, [x], np.zeros((C, R), dtype), {"R": R, "C": C}, WARP_ROWS=warp_rows, CTAS_PER_SM=4)
        assert out.tobytes() == want, (R, C, "blocks")
        out = run(rt, spec, [x], np.zeros((C, R), dtype), {"R": R, "C": C}, WARP_ROWS=warp_rows, TILE_ORDER=1)
        assert out.tobytes() == want, (R, C, "diagonal tile order")
        out = run(rt, spec, [x], np.zeros((C, R), dtype), {"R": R, "C": C}, WARP_ROWS=warp_rows, TILE_ORDER=2)
        assert out.tobytes() == want, (R, C, "column-major tile order")
        for variant in (1, 2, 3):
            out = run(rt, spec, [x], np.zeros((C, R), dtype), {"R": R, "C": C}, WARP_ROWS=warp_rows, VARIANT=variant)
            assert out.tobytes() == want, (R, C, "variant", variant)
        out = run(rt, spec, [x], np.zeros((C, R), dtype), {"R": R, "C": C}, TILE_KERNEL=1)
        assert out.tobytes() == want, (R, C, "tiles")


@pytest.mark.parametrize("R,C", [(64, 64), (512, 256), (520, 264), (8, 8), (1000, 24), (24, 1000), (4104, 600), (72, 4104)])
def test_transpose_2d_copy_engine_kernel(rt, R, C):
    """The copy-engine transpose (tensor-map loads, ldmatrix.trans / stmatrix, tensor-map stores; 16-bit elements,
    asked for with VARIANT=4): whole tiles, tiles ragged in either direction (loads past the edge read zeros, stores are
    clipped), a matrix smaller than one tile, more tiles than CTAs (its tiles are walked in squares of 8 x 8, whose
    border squares hold tiles that lie outside the matrix)."""
    rng = np.random.default_rng(R + C)
    x = rng.standard_normal((R, C)).astype(np.float16)
    want = oracle.transpose_2d(x).tobytes()
    spec = descriptors.transpose_2d("f16")
    out = run(rt, spec, [x], np.full((C, R), np.float16(7), np.float16), {"R": R, "C": C}, VARIANT=4)
    assert out.tobytes() == want, "copy engine"
    # 32-bit elements have no copy-engine kernel: the hint falls back to the register blocks
    x32 = x.astype(np.float32)
    out = run(rt, descriptors.transpose_2d("f32"), [x32], np.zeros((C, R), np.float32), {"R": R, "C": C}, VARIANT=4)
    assert out.tobytes() == oracle.transpose_2d(x32).tobytes()


def test_transpose_2d_round_trip_at_full_size(rt):
    """Size-independent property at the bench shape: transposing twice gives the input back, bit for bit."""
    rng = np.random.default_rng(12)
    x = rng.standard_normal((8192, 8192), dtype=np.float32).astype(np.float16)
    spec = descriptors.transpose_2d("f16")
    once = run(rt, spec, [x], np.zeros((8192, 8192), np.float16), {"R": 8192, "C": 8192})
    assert once[5, 7] == x[7, 5] and once[8191, 0] == x[0, 8191]
    twice = run(rt, spec, [once], np.zeros((8192, 8192), np.float16), {"R": 8192, "C": 8192})
    assert twice.tobytes() == x.tobytes()


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("M,N", [(512, 256), (520, 264), (8, 8), (1000, 24), (24, 1000), (3, 5), (257, 129)])
def test_elementwise_with_a_transposed_operand(rt, dtype, M, N):
    """out[n, m] = (a[m, n] + b[n, m]) * c[n], rounding after every op: whole blocks, ragged blocks, shapes whose
    strides are not multiples of 16 bytes (those take the element-wise kernel), all against numpy."""
    rng = np.random.default_rng(21)
    a = rng.standard_normal((M, N)).astype(dtype)
    b = rng.standard_normal((N, M)).astype(dtype)
    c = rng.standard_normal(N).astype(dtype)
    want = ((a.T + b).astype(dtype) * c[:, None]).astype(dtype)
    spec = descriptors.transposed_add_mul("f16" if dtype == np.float16 else "f32")
    out = run(rt, spec, [a, b, c], np.zeros((N, M), dtype), {"M": M, "N": N})
    assert out.tobytes() == want.tobytes()


@pytest.mark.parametrize("B,M,N", [(3, 128, 64), (2, 100, 36), (1, 4, 4), (5, 33, 7)])
def test_batched_transposed_operand_with_interpreted_body(rt, B, M, N):
    rng = np.random.default_rng(22)
    a = rng.standard_normal((B, M, N)).astype(np.float32)
    bias = rng.standard_normal(M).astype(np.float32)
    want = (np.maximum(a, np.float32(0)).transpose(0, 2, 1) - bias[None, None, :]).astype(np.float32)
    spec = descriptors.batched_transposed_relu_sub("f32")
    out = run(rt, spec, [a, bias], np.zeros((B, N, M), np.float32), {"B": B, "M": M, "N": N})
    assert out.tobytes() == np.ascontiguousarray(want).tobytes()


def test_interpreted_body_matches_oracle_chain(rt):
    # a chain with no straight-line specialisation: ((a - b) / b) min a
    spec = descriptors.add_mul()
    import copy
    d = copy.deepcopy(spec.descriptor)
    d["kernel"] = "sub_div_min"
    d["body"] = [descriptors.op("subf", "v0", "v1"), descriptors.op("divf", "%0", "v1"), descriptors.op("minimumf", "%1", "v0")]
    rng = np.random.default_rng(8)
    a = rng.uniform(-1, 1, (33, 64)).astype(np.float32)
    b = rng.uniform(0.5, 1.5, (33, 64)).astype(np.float32)
    out = np.zeros_like(a)
    rt.run(descriptors.container(d), "sub_div_min", [a, b], [out], spec.pack({"M": 33, "N": 64}))
    assert np.array_equal(out, np.minimum((a - b) / b, a))


# ---- row reduction ------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N", [(256, 8192), (7, 33), (1, 1), (300, 1000), (4, 65536), (1000, 32)])
def test_bcast_add_rowsum_f32_within_bound(rt, M, N):
    w = configs.broadcast_add_reduce(M, N, seed=9)
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape)
    ref, s64, abs64 = oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1], with_bounds=True)
    # |gpu - exact| <= 1e-5 * sum|x_ij + b_i|; the sequential CPU sum sits inside the same bound
    assert np.all(np.abs(out - s64) <= 1e-5 * abs64 + 1e-30)
    assert np.all(np.abs(ref - s64) <= 1e-5 * abs64 + 1e-30)


@pytest.mark.parametrize("split", [1, 2, 5, 16])
def test_rowsum_split_columns_use_workspace(rt, split):
    w = configs.broadcast_add_reduce(5, 40000, seed=10)
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape, SPLIT_N=split)
    assert rt.last_launch_count == (2 if split > 1 else 1)
    _, s64, abs64 = oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1], with_bounds=True)
    assert np.all(np.abs(out - s64) <= 1e-5 * abs64)


def test_reference_reduce_example_golden(rt, golden_dir):
    g = dict(np.load(golden_dir / "broadcast_add_reduce.npz"))
    spec = descriptors.bcast_add_rowsum("f16")
    M, N = g["input_b"].shape
    out = run(rt, spec, [g["input_a"], g["input_b"]], np.zeros(M, np.float16), {"M": M, "N": N})
    want = oracle.bcast_add_rowsum_f16(g["input_a"], g["input_b"])
    # f32 accumulation order differs; after the final f16 rounding at most one ulp apart
    assert np.max(np.abs(out.astype(np.float32) - want.astype(np.float32))) <= np.max(np.abs(want.astype(np.float32))) * 2.0 ** -10
    fails, _, _ = oracle.compare(out.astype(np.float32), g["output_c"].astype(np.float32), 10.0, 1e-2)
    assert fails == 0


# ---- gather ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,W,R", [(4096, 256, 2048), (100, 8, 33), (50, 7, 20), (10, 256, 1), (65536, 64, 5000)])
def test_gather_rows_bf16_bit_exact(rt, T, W, R):
    w = configs.gather_elementwise(T, W, R, seed=11)
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape)
    assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs))


def test_gather_rows_edges_and_duplicates(rt):
    w = configs.gather_elementwise(1000, 64, 512, seed=12)
    idx = w.inputs[1]
    idx[:4] = [0, 999, 0, 999]
    idx[100:200] = idx[300]  # heavy duplication
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape)
    assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs))


def test_gather_rows_out_of_range_index_is_reported_not_clamped(rt):
    w = configs.gather_elementwise(100, 16, 40, seed=13)
    w.inputs[1][7] = 100
    w.inputs[1][9] = -1
    out = np.full(w.out_shape, 0x7FC0, np.uint16)
    with pytest.raises(ExecutorError, match=r"gather index out of range \(2 indices\)"):
        rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling())
    # the context survives and the next call works
    w.inputs[1][[7, 9]] = 0
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape)
    assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs))


@pytest.mark.parametrize("T,W,R,tile", [
    (5000, 256, 40003, {"BULK_COPY": 1}),                     # default ring: 8 rows per stage, ragged last chunk
    (70000, 64, 80001, {"BULK_COPY": 1}),                     # 128-byte rows: 32 rows per stage
    (5000, 256, 40003, {"BULK_COPY": 1, "STREAM_STAGES": 2, "STREAM_ROWS": 4}),
    (5000, 256, 40003, {"BULK_COPY": 1, "STREAM_STAGES": 6, "STREAM_ROWS": 2}),
    (3000, 512, 30001, {"BULK_COPY": 1, "STREAM_STAGES": 4, "STREAM_ROWS": 16}),
    (5000, 256, 80001, {"BULK_COPY": 1, "STREAM_STAGES": 3, "STREAM_ROWS": 4, "STREAM_WARPS": 16}),
    (9000, 128, 160001, {"BULK_COPY": 1, "STREAM_WARPS": 4}),  # rows shorter than a warp of vectors
    (5000, 256, 40003, {}),                                   # same shapes on the default plain-load kernel
])
def test_gather_rows_staged_kernel_bit_exact(rt, monkeypatch, T, W, R, tile):
    """The opt-in bulk-copy staged kernel at shapes large enough for it, whole launch (the host path is told not
    to cut the rows into chunks, which would fall below the kernel's size threshold)."""
    monkeypatch.setenv("AFIR_CUDA_NO_PIPELINE", "1")
    w = configs.gather_elementwise(T, W, R, seed=14)
    w.inputs[1][:6] = [0, T - 1, 0, T - 1, 17, 17]
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape, **tile)
    assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs))


def test_gather_rows_staged_kernel_i64_indices_and_bad_indices(rt, monkeypatch):
    monkeypatch.setenv("AFIR_CUDA_NO_PIPELINE", "1")
    w = configs.gather_elementwise(5000, 256, 40003, seed=15)
    spec = descriptors.gather_rows_scale_resid("bf16", "i64")
    inputs = [w.inputs[0], w.inputs[1].astype(np.int64), w.inputs[2], w.inputs[3]]
    want = oracle.gather_rows_scale_resid_bf16(*w.inputs)
    out = run(rt, spec, inputs, w.new_output(), w.shape, BULK_COPY=1)
    assert np.array_equal(out, want)
    # out-of-range indices in the middle of a stage and in the ragged last chunk: counted; the other rows are right
    bad_rows = [11, 12, 20001, 40002]
    inputs[1][bad_rows] = [5000, -3, 1 << 40, 5000]
    out = np.full(w.out_shape, 0x7FC0, np.uint16)
    with pytest.raises(ExecutorError, match=r"gather index out of range \(4 indices\)"):
        rt.run(spec.binary, spec.name, inputs, [out], spec.pack(w.shape, BULK_COPY=1))
    keep = np.ones(40003, bool)
    keep[bad_rows] = False
    assert np.array_equal(out[keep], want[keep])
    inputs[1][bad_rows] = 0
    out = run(rt, spec, inputs, w.new_output(), w.shape, BULK_COPY=1)
    assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(inputs[0], inputs[1].astype(np.int32), inputs[2], inputs[3]))


def test_reference_gather_example_golden_exact(rt, golden_dir):
    g = dict(np.load(golden_dir / "gather_elementwise_fusion.npz"))
    spec = descriptors.relu_gather_cols_bias()
    M, N = g["input_data"].shape
    K = g["input_indices"].shape[0]
    out = run(rt, spec, [g["input_data"], g["input_indices"], g["input_bias"]], np.zeros((M, K), np.float16),
              {"M": M, "N": N, "K": K})
    assert out.tobytes() == g["output_out"].tobytes()


def test_gather_cols_i32_and_odd_shapes(rt):
    rng = np.random.default_rng(14)
    data = rng.standard_normal((37, 91)).astype(np.float16)
    idx = rng.integers(0, 91, 53).astype(np.int32)
    bias = rng.standard_normal(53).astype(np.float16)
    spec = descriptors.relu_gather_cols_bias("f16", "i32")
    out = run(rt, spec, [data, idx, bias], np.zeros((37, 53), np.float16), {"M": 37, "N": 91, "K": 53})
    assert np.array_equal(bits(out), bits(oracle.relu_gather_cols_bias_f16(data, idx.astype(np.int64), bias)))


# ---- shape errors surface before any launch -------------------------------------------------------------------
def test_byte_size_mismatch_is_refused(rt):
    w = configs.elementwise_chain(8, 16)
    with pytest.raises(ExecutorError, match="bytes, the tiling dims imply"):
        rt.run(w.spec.binary, w.spec.name, w.inputs, [w.new_output()], w.spec.pack({"M": 8, "N": 32}))


def test_run_file_matches_run(rt, tmp_path):
    w = configs.elementwise_chain(64, 64, seed=15)
    p = tmp_path / "k.bin"
    p.write_bytes(w.spec.binary)
    out = w.new_output()
    rt.run_file(str(p), w.spec.name, w.inputs, [out], w.tiling())
    assert np.array_equal(out, oracle.add_mul_f32(*w.inputs))


# ---- matmul + bias + LeakyReLU (tcgen05) ---------------------------------------------------------------------
def _matmul_check(rt, M, N, K, mb, seed=0):
    w = configs.matmul_add_leakyrelu(M, N, K, seed=seed)
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape, STAGES=mb)
    got = oracle.bf16_to_f32(out)
    want = oracle.bf16_to_f32(oracle.matmul_bias_leakyrelu_bf16(*w.inputs, 0.01))
    # bar: relative error <= 1e-2 (bf16 output rounding alone is 2^-9); tiny absolute floor for values near zero
    assert np.all(np.abs(got - want) <= 1e-2 * np.abs(want) + 1e-3)
    # and tight in aggregate: at most one bf16 ulp apart almost everywhere
    assert np.mean(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-6) > 0.999


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 320), (100, 136, 72), (1, 8, 8),
                                   (130, 264, 1032), (1024, 1024, 1024)])
@pytest.mark.parametrize("mb", [1, 2, 3])
def test_matmul_bias_leakyrelu_bf16(rt, M, N, K, mb):
    _matmul_check(rt, M, N, K, mb, seed=M + N + K)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (384, 768, 320), (100, 136, 72), (1, 8, 8), (130, 264, 1032), (1024, 1024, 1024),
                                   (2048, 4096, 512)])
@pytest.mark.parametrize("mb", [1, 2, 3])
def test_matmul_with_b_given_as_n_by_k(rt, M, N, K, mb):
    """out = A x B^T with B stored [N, K] (the layout of a torch Linear weight): the kernel loads K-major tiles of it.
    Same oracle, fed the transpose; the two layouts must also agree with each other bit for bit (same products,
    same accumulation order in the tensor core).  STAGES=3 asks for the CTA-pair kernel, which this layout
    replaces by the single-CTA one."""
    w = configs.matmul_add_leakyrelu(M, N, K, seed=M + N + K + 1)
    a, b, bias = w.inputs
    bt = np.ascontiguousarray(b.T)
    spec_t = descriptors.matmul_bias_leakyrelu(transpose_b=True)
    out_t = run(rt, spec_t, [a, bt, bias], w.new_output(), w.shape, STAGES=mb)
    got = oracle.bf16_to_f32(out_t)
    want = oracle.bf16_to_f32(oracle.matmul_bias_leakyrelu_bf16(a, b, bias, 0.01))
    assert np.all(np.abs(got - want) <= 1e-2 * np.abs(want) + 1e-3)
    assert np.mean(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-6) > 0.999
    out_n = run(rt, w.spec, w.inputs, w.new_output(), w.shape, STAGES=min(mb, 2))
    assert np.array_equal(out_t.view(np.uint16), out_n.view(np.uint16))


def test_launch_trace_carries_the_matmul_plan(rt, monkeypatch, capfd):
    """With launch tracing on, the planner's one-line description of what was launched follows the argument lines."""
    monkeypatch.setenv("AFIR_CUDA_TRACE_LAUNCH", "1")
    w = configs.matmul_add_leakyrelu(384, 768, 320, seed=5)
    run(rt, w.spec, w.inputs, w.new_output(), w.shape)
    err = capfd.readouterr().err
    assert "[cuda-launch] kernel=matmul_add_leakyrelu " in err
    plan = [l for l in err.splitlines() if "matmul plan" in l]
    assert plan and "variant=rows128" in plan[0] and "tile=128x256x64" in plan[0] and "tiles=3x3" in plan[0] and "k_blocks=5" in plan[0]
    assert "planned_block_dim=9 " in plan[0]


def test_matmul_many_tiles_per_cta(rt):
    # more tiles than SMs: every CTA walks several tiles, both TMEM accumulators and all ring phases wrap
    _matmul_check(rt, 2048, 4096, 512, 1, seed=21)
    _matmul_check(rt, 4096, 4096, 256, 2, seed=22)
    _matmul_check(rt, 4096, 2048, 512, 3, seed=25)
    _matmul_check(rt, 2000, 1032, 264, 3, seed=26)


@pytest.mark.parametrize("tile_n", [128, 160, 192, 224, 256])
@pytest.mark.parametrize("mb", [1, 2])
def test_matmul_tile_widths(rt, monkeypatch, tile_n, mb):
    """The CTA tile can be narrower than 256 columns (224 ... 128, a planner hint); every width must give the same
    result: ragged N (1000 is not a multiple of any width), several tiles per CTA, both layouts of B."""
    monkeypatch.setenv("AFIR_GEMM_TILE_N", str(tile_n))
    _matmul_check(rt, 520, 1000, 320, mb, seed=tile_n + mb)
    _matmul_check(rt, 2048, 4096, 256, mb, seed=tile_n)
    w = configs.matmul_add_leakyrelu(300, 1000, 128, seed=tile_n)
    spec = descriptors.matmul_bias_leakyrelu(transpose_b=True)
    A, B, bias = w.inputs
    out = run(rt, spec, [A, np.ascontiguousarray(B.T), bias], w.new_output(), w.shape, STAGES=mb)
    assert np.array_equal(out, run(rt, w.spec, w.inputs, w.new_output(), w.shape, STAGES=mb))


def test_matmul_m_sharded_shapes(rt):
    """8192^3 M-sharded over 8 and 4 GPUs is M = 1024 and 2048 per GPU (fewer tiles than two waves of SMs)."""
    _matmul_check(rt, 1024, 8192, 512, 0, seed=77)
    _matmul_check(rt, 2048, 8192, 256, 0, seed=78)


def test_reference_matmul_example_golden_max_abs_diff_zero(rt, golden_dir):
    g = dict(np.load(golden_dir / "matmul_add_leakyrelu.npz"))
    spec = descriptors.matmul_bias_leakyrelu("f16", "f32", "f32", alpha=0.001)
    M, K = g["input_a"].shape
    N = g["input_b"].shape[1]
    out = run(rt, spec, [g["input_a"], g["input_b"], g["input_bias"]], np.zeros((M, N), np.float32), {"M": M, "N": N, "K": K})
    # integer-valued operands: every partial sum is exact, so the tensor-core result equals the golden
    # wherever the epilogue is the identity, and differs by one f32 rounding of alpha*x elsewhere
    pos = g["output"] >= 0
    assert np.array_equal(out[pos], g["output"][pos])
    assert np.max(np.abs(out - g["output"])) <= 1e-6 * np.max(np.abs(g["output"]))
    want = oracle.matmul_bias_leakyrelu_f16_f32(g["input_a"], g["input_b"], g["input_bias"], 0.001)
    assert np.array_equal(out, want)  # against the oracle (same f32 alpha): max_abs_diff == 0


@pytest.mark.parametrize("epilogue", ["None", "BiasAdd", "BiasAddRelu"])
def test_matmul_other_epilogues(rt, epilogue):
    rng = np.random.default_rng(23)
    M, N, K = 192, 320, 128
    A = rng.integers(-4, 5, (M, K)).astype(np.float16)
    B = rng.integers(-4, 5, (K, N)).astype(np.float16)
    bias = rng.integers(-8, 9, N).astype(np.float32)
    spec = descriptors.matmul_bias_leakyrelu("f16", "f32", "f32", alpha=0.0, epilogue=epilogue)
    out = run(rt, spec, [A, B, bias], np.zeros((M, N), np.float32), {"M": M, "N": N, "K": K})
    x = A.astype(np.float32) @ B.astype(np.float32)
    if epilogue != "None":
        x = x + bias
    if epilogue == "BiasAddRelu":
        x = np.maximum(x, 0)
    assert np.array_equal(out, x)


def test_matmul_refuses_rows_tma_cannot_address(rt):
    w = configs.matmul_add_leakyrelu(64, 64, 36)
    with pytest.raises(ExecutorError, match="multiples of 8"):
        rt.run(w.spec.binary, w.spec.name, w.inputs, [w.new_output()], w.tiling())


def test_matmul_linearity_at_scale(rt):
    # size-independent property at a size the CPU oracle would take minutes for:
    # with epilogue None, (2A).B == 2 (A.B) exactly (power-of-two scaling commutes with every rounding)
    rng = np.random.default_rng(24)
    M = N = K = 2048
    A = configs.f32_to_bf16_bits(rng.standard_normal((M, K), dtype=np.float32) * np.float32(0.02))
    B = configs.f32_to_bf16_bits(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
    A2 = configs.f32_to_bf16_bits(configs.bf16_bits_to_f32(A) * np.float32(2))
    bias = np.zeros(N, np.uint16)
    spec = descriptors.matmul_bias_leakyrelu("bf16", "bf16", "bf16", alpha=0.0, epilogue="None")
    shape = {"M": M, "N": N, "K": K}
    o1 = run(rt, spec, [A, B, bias], np.zeros((M, N), np.uint16), shape)
    o2 = run(rt, spec, [A2, B, bias], np.zeros((M, N), np.uint16), shape)
    assert np.array_equal(configs.bf16_bits_to_f32(o2), configs.bf16_bits_to_f32(o1) * np.float32(2))
    # sampled f64 check of the fused form
    w_bias = configs.f32_to_bf16_bits(rng.standard_normal(N, dtype=np.float32) * np.float32(0.1))
    spec2 = descriptors.matmul_bias_leakyrelu()
    o3 = configs.bf16_bits_to_f32(run(rt, spec2, [A, B, w_bias], np.zeros((M, N), np.uint16), shape))
    for m, n in rng.integers(0, M, (64, 2)):
        want = oracle.matmul_bias_leakyrelu_bf16_at(A, B, w_bias, 0.01, int(m), int(n))
        assert abs(o3[m, n] - want) <= 1e-2 * abs(want) + 1e-3


# ---- integer element types ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,name", [(np.int32, "i32"), (np.int16, "i16")])
@pytest.mark.parametrize("M,N", [(64, 256), (33, 1000), (7, 5), (1, 1)])
def test_integer_elementwise_wraps_like_twos_complement(rt, dtype, name, M, N):
    """afir.add then afir.mul on integer tensors: (a + b) * b with wrap-around, over the whole value range."""
    rng = np.random.default_rng(41)
    info = np.iinfo(dtype)
    a = rng.integers(info.min, info.max, (M, N), dtype=dtype, endpoint=True)
    b = rng.integers(info.min, info.max, (M, N), dtype=dtype, endpoint=True)
    with np.errstate(over="ignore"):
        want = ((a + b) * b).astype(dtype)
    out = run(rt, descriptors.add_mul(name), [a, b], np.zeros((M, N), dtype), {"M": M, "N": N})
    assert np.array_equal(out, want)


@pytest.mark.parametrize("dtype,name", [(np.int32, "i32"), (np.int16, "i16")])
def test_integer_body_ops_division_max_min_constants_and_a_transposed_operand(rt, dtype, name):
    rng = np.random.default_rng(42)
    M, N = 520, 264
    a = rng.integers(-1000, 1000, (M, N)).astype(dtype)
    b = rng.integers(-50, 50, (N, M)).astype(dtype)
    b[b == 0] = 7
    a[0, 0], b[0, 0] = np.iinfo(dtype).min, -1
    # out[n, m] = min(max(a[m, n], -100) / b[n, m] - 3, 40): truncating division, constants, a transposed read
    dims = [("dim_arg0_0", "M"), ("dim_arg0_1", "N")]
    dom = ["dim_arg0_1", "dim_arg0_0"]
    body = {"domain": dom,
            "loads": [{"arg": 0, "shape": ["dim_arg0_0", "dim_arg0_1"], "map": [1, 0]}, {"arg": 1, "shape": dom, "map": [0, 1]}],
            "store": {"arg": 2, "shape": dom, "map": [0, 1]},
            "body": [descriptors.op("maxsi", "v0", -100), descriptors.op("divsi", "%0", "v1"), descriptors.op("subi", "%1", 3),
                     descriptors.op("minsi", "%2", 40)]}
    spec = descriptors._spec("int_chain", "elementwise", name, 2, 1, descriptors._EW_TILE, dims, body, descriptors._EW_LAUNCH)
    t = np.maximum(a.T.astype(np.int64), -100)
    q = np.trunc(t / b.astype(np.int64)).astype(np.int64)  # C-style truncation toward zero
    want = np.minimum(q - 3, 40).astype(dtype)
    out = run(rt, spec, [a, b], np.zeros((N, M), dtype), {"M": M, "N": N})
    assert np.array_equal(out, want)
    # same chain on a ragged shape (element-wise path)
    a2, b2 = np.ascontiguousarray(a[:37, :29]), np.ascontiguousarray(b[:29, :37])
    out = run(rt, spec, [a2, b2], np.zeros((29, 37), dtype), {"M": 37, "N": 29})
    t = np.maximum(a2.T.astype(np.int64), -100)
    assert np.array_equal(out, np.minimum(np.trunc(t / b2.astype(np.int64)).astype(np.int64) - 3, 40).astype(dtype))


@pytest.mark.parametrize("M,N", [(7, 5), (33, 37), (64, 256)])
def test_int16_add_sub_max_min_one_element_at_a_time_and_in_vectors(rt, M, N):
    """((a + 3) - b, max with -7, + b, - 5, min with 1000) on int16 over the whole value range, with wrap-around: on
    ragged shapes the kernels evaluate the two-lane pack on one splatted element and keep its low lane, a context in
    which the compiler's two-lane add / subtract intrinsics came back wrong, so the pack spells the arithmetic out."""
    rng = np.random.default_rng(43)
    info = np.iinfo(np.int16)
    a = rng.integers(info.min, info.max, (M, N), dtype=np.int16, endpoint=True)
    b = rng.integers(info.min, info.max, (M, N), dtype=np.int16, endpoint=True)
    spec = descriptors.add_mul("i16")
    d = copy.deepcopy(spec.descriptor)
    d["kernel"] = "int16_lanes"
    d["body"] = [descriptors.op("addi", "v0", 3), descriptors.op("subi", "%0", "v1"), descriptors.op("maxsi", "%1", -7),
                 descriptors.op("addi", "%2", "v1"), descriptors.op("subi", "%3", 5), descriptors.op("minsi", "%4", 1000)]
    out = np.zeros((M, N), np.int16)
    rt.run(descriptors.container(d), d["kernel"], [a, b], [out], spec.pack({"M": M, "N": N}))
    with np.errstate(over="ignore"):
        t = np.maximum(((a + np.int16(3)).astype(np.int16) - b).astype(np.int16), np.int16(-7))
        want = np.minimum(((t + b).astype(np.int16) - np.int16(5)).astype(np.int16), np.int16(1000))
    assert np.array_equal(out, want)


def test_integer_division_by_zero_is_defined_as_zero(rt):
    a = np.array([[5, -7, 0, 9]], np.int32)
    b = np.array([[0, 0, 0, 3]], np.int32)
    dims = [("dim_arg0_0", "M"), ("dim_arg0_1", "N")]
    shp = ["dim_arg0_0", "dim_arg0_1"]
    view = lambda arg: {"arg": arg, "shape": shp, "map": [0, 1]}  # noqa: E731
    body = {"domain": shp, "loads": [view(0), view(1)], "store": view(2), "body": [descriptors.op("divsi", "v0", "v1")]}
    spec = descriptors._spec("int_div", "elementwise", "i32", 2, 1, descriptors._EW_TILE, dims, body, descriptors._EW_LAUNCH)
    out = run(rt, spec, [a, b], np.zeros((1, 4), np.int32), {"M": 1, "N": 4})
    assert out.tolist() == [[0, 0, 0, 3]]


def test_integer_transpose_and_unsupported_classes(rt):
    x = np.arange(520 * 264, dtype=np.int32).reshape(520, 264)
    out = run(rt, descriptors.transpose_2d("i32"), [x], np.zeros((264, 520), np.int32), {"R": 520, "C": 264})
    assert np.array_equal(out, x.T)
    w = configs.broadcast_add_reduce(8, 16)
    spec = descriptors.bcast_add_rowsum("i32")
    with pytest.raises(ExecutorError, match="f32, f16 or bf16"):
        rt.run(spec.binary, spec.name, [w.inputs[0].view(np.int32), w.inputs[1].view(np.int32)], [np.zeros(8, np.int32)],
               spec.pack({"M": 8, "N": 16}))


# ---- guard bands -------------------------------------------------------------------------------------------------
def test_no_kernel_writes_outside_its_output_at_ragged_shapes(rt, monkeypatch):
    """With AFIR_CUDA_CANARY=1 every host-path buffer sits between two 4 KB bands of a known pattern and the bands of
    the outputs are checked after the run: one ragged shape per kernel class (and per variant that has its own
    store code) must leave them intact and still give the oracle's result."""
    monkeypatch.setenv("AFIR_CUDA_CANARY", "1")
    rng = np.random.default_rng(31)

    w = configs.elementwise_chain(257, 1023, seed=31)
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape)
    assert np.array_equal(out, oracle.add_mul_f32(*w.inputs))

    w = configs.split_relu_broadcast_add_mul(3, 37, 72, seed=31)
    out = run(rt, w.spec, w.inputs, w.new_output(), w.shape)
    assert np.array_equal(bits(out), bits(oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], 1)))

    w = configs.broadcast_add_reduce(1501, 4100, seed=31)
    for tile in ({}, {"BULK_COPY": 0}, {"BULK_COPY": 0, "SPLIT_N": 4}):
        out = run(rt, w.spec, w.inputs, w.new_output(), w.shape, **tile)
        _, s64, abs64 = oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1], with_bounds=True)
        assert np.all(np.abs(out - s64) <= 1e-5 * abs64), tile

    monkeypatch.setenv("AFIR_CUDA_NO_PIPELINE", "1")
    w = configs.gather_elementwise(5000, 256, 40003, seed=31)
    for tile in ({}, {"BULK_COPY": 1}):
        out = run(rt, w.spec, w.inputs, w.new_output(), w.shape, **tile)
        assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs)), tile
    monkeypatch.delenv("AFIR_CUDA_NO_PIPELINE")

    x = rng.standard_normal((1001, 523)).astype(np.float16)
    spec = descriptors.transpose_2d("f16")
    for tile in ({}, {"TILE_KERNEL": 1}, {"VARIANT": 3}):
        out = run(rt, spec, [x], np.zeros((523, 1001), np.float16), {"R": 1001, "C": 523}, **tile)
        assert out.tobytes() == oracle.transpose_2d(x).tobytes(), tile
    x = rng.standard_normal((1000, 520)).astype(np.float16)
    out = run(rt, spec, [x], np.zeros((520, 1000), np.float16), {"R": 1000, "C": 520})
    assert out.tobytes() == oracle.transpose_2d(x).tobytes()

    a = rng.standard_normal((1000, 264)).astype(np.float16)
    b = rng.standard_normal((264, 1000)).astype(np.float16)
    c = rng.standard_normal(264).astype(np.float16)
    out = run(rt, descriptors.transposed_add_mul("f16"), [a, b, c], np.zeros((264, 1000), np.float16), {"M": 1000, "N": 264})
    assert out.tobytes() == ((a.T + b).astype(np.float16) * c[:, None]).astype(np.float16).tobytes()

    for mb in (1, 2, 3):
        w = configs.matmul_add_leakyrelu(300, 264, 136, seed=31)
        out = run(rt, w.spec, w.inputs, w.new_output(), w.shape, STAGES=mb)
        got = oracle.bf16_to_f32(out)
        want = oracle.bf16_to_f32(oracle.matmul_bias_leakyrelu_bf16(*w.inputs, 0.01))
        assert np.all(np.abs(got - want) <= 1e-2 * np.abs(want) + 1e-3), mb
