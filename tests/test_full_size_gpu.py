"""The five benchmark configurations at their FULL sizes through afirt_executor_run (host buffers, so the chunked
copy/compute pipeline is exercised too): groups 1-4 are compared element for element with the CPU oracle, which is
fast enough at these sizes; the 8192^3 GEMM is checked on 160 whole rows (f32-accumulating oracle), on the exact
power-of-two linearity of the unfused product, and on a column checksum against those rows' contributions."""
import numpy as np
import pytest

from ascend_mlir_b200 import build as lib_build
from ascend_mlir_b200 import configs, descriptors
from ascend_mlir_b200.runtime import CudaRuntime
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    lib_build.build()
    r = CudaRuntime()
    r.set_device(0)
    return r


def run(rt, w, **tile):
    out = w.new_output()
    rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling(**tile), block_dim=0, magic=w.spec.magic)
    return out


def test_config1_elementwise_chain_full_size_bit_exact(rt):
    w = configs.elementwise_chain()
    assert w.inputs[0].shape == (4096, 4096)
    out = run(rt, w)
    assert np.array_equal(out.view(np.uint32), oracle.add_mul_f32(*w.inputs).view(np.uint32))


def test_config2_split_relu_broadcast_add_mul_full_size_bit_exact(rt):
    w = configs.split_relu_broadcast_add_mul()
    assert w.inputs[0].shape == (32, 1024, 2048) and w.out_shape == (32, 1024, 1024)
    out = run(rt, w)
    want = oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], 1)
    assert np.array_equal(out.view(np.uint16), want.view(np.uint16))


def test_config3_broadcast_add_reduce_full_size_within_bound(rt):
    w = configs.broadcast_add_reduce()
    assert w.inputs[1].shape == (8192, 8192)
    out = run(rt, w)
    cpu, s64, abs64 = oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1], with_bounds=True)
    assert np.all(np.abs(out - s64) <= 1e-5 * abs64)
    assert np.all(np.abs(cpu - s64) <= 1e-5 * abs64), "the sequential CPU order sits inside the same bound"


def test_config4_gather_elementwise_full_size_bit_exact(rt):
    w = configs.gather_elementwise()
    assert w.inputs[0].shape == (1048576, 256) and w.inputs[1].shape == (262144,) and w.inputs[1].dtype == np.int32
    uniq = np.unique(w.inputs[1]).size
    assert 0.04 <= 1 - uniq / w.inputs[1].size <= 0.06, "about 5 % duplicate indices"
    out = run(rt, w)
    assert np.array_equal(out, oracle.gather_rows_scale_resid_bf16(*w.inputs))


def test_config5_matmul_add_leakyrelu_full_size(rt):
    w = configs.matmul_add_leakyrelu()
    A, B, bias = w.inputs
    assert A.shape == B.shape == (8192, 8192) and bias.shape == (8192,)
    out = configs.bf16_bits_to_f32(run(rt, w))
    rng = np.random.default_rng(5)
    rows = np.unique(np.concatenate([np.arange(32), np.arange(8160, 8192), rng.integers(32, 8160, 96)]))
    want = configs.bf16_bits_to_f32(oracle.matmul_bias_leakyrelu_bf16(np.ascontiguousarray(A[rows]), B, bias, 0.01))
    got = out[rows]
    assert np.all(np.abs(got - want) <= 1e-2 * np.abs(want) + 1e-3)
    assert np.mean(got == want) > 0.99, "all but a few elements agree to the last bf16 bit"
    # every column's checksum over the sampled rows, accumulated in f64 on both sides
    assert np.allclose(got.astype(np.float64).sum(axis=0), want.astype(np.float64).sum(axis=0), rtol=1e-3, atol=1e-2)

    # EVERY element of the 8192 x 8192 result against an f32 matmul on the CPU (torch: A.B in f32 from the exact bf16
    # operands, + bias, max(x, 0.01 x), rounded once to bf16), within 1e-2 relative: a tile dropped or misplaced
    # anywhere in the matrix shows here; the 160 oracle rows above stay the tight, order-exact check
    import torch
    a32 = torch.from_numpy(configs.bf16_bits_to_f32(A))
    b32 = torch.from_numpy(configs.bf16_bits_to_f32(B))
    x = a32 @ b32 + torch.from_numpy(configs.bf16_bits_to_f32(bias))[None, :]
    full = torch.maximum(x, x * 0.01).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.all(np.abs(out - full) <= 1e-2 * np.abs(full) + 1e-3), "full-matrix comparison"
    assert np.mean(np.abs(out - full) <= 2.0 ** -7 * np.abs(full) + 1e-6) > 0.999
    del a32, b32, x, full

    # linearity of the unfused product at full size: (2A).B == 2 (A.B) bit for bit
    spec = descriptors.matmul_bias_leakyrelu("bf16", "bf16", "bf16", alpha=0.0, epilogue="None")
    shape = {"M": 8192, "N": 8192, "K": 8192}
    A2 = configs.f32_to_bf16_bits(configs.bf16_bits_to_f32(A) * np.float32(2))
    o1, o2 = np.zeros((8192, 8192), np.uint16), np.zeros((8192, 8192), np.uint16)
    rt.run(spec.binary, spec.name, [A, B, bias], [o1], spec.pack(shape), block_dim=0, magic=spec.magic)
    rt.run(spec.binary, spec.name, [A2, B, bias], [o2], spec.pack(shape), block_dim=0, magic=spec.magic)
    assert np.array_equal(configs.bf16_bits_to_f32(o2), configs.bf16_bits_to_f32(o1) * np.float32(2))
