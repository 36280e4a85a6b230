"""Pins the CPU oracle against the reference's own numpy goldens.

The .npz fixtures were written by the reference's examples/*/gen_data.py
scripts (tests/golden/make_golden.py).  Tolerances are the ones each
reference run.sh passes to its validator: split atol=rtol=1e-2
(examples/split-relu-brc-add-mul/run.sh:207-208), reduce and gather atol=10,
rtol=1e-2 (examples/broadcast-add-reduce/run.sh:262-263), matmul must print
max_abs_diff=0 (test/tools/examples/example_pipelines.sh:139-147), transpose is
memcmp-exact (test/tools/runtime/test_capi_runtime.cpp:178).
"""
import numpy as np
import pytest

from oracle import oracle


def _load(golden_dir, name):
    return dict(np.load(golden_dir / f"{name}.npz"))


def test_f16_bf16_known_answers():
    # known answers the reference's npy tests use: f16 1.0 = 0x3C00, bf16 1.0 = 0x3F80
    # (test/tools/runtime/test_runtime.cpp:169-281)
    assert oracle.f32_to_f16_bits(np.array([1.0], np.float32))[0] == 0x3C00
    assert oracle.f32_to_bf16(np.array([1.0], np.float32))[0] == 0x3F80
    assert oracle.bf16_to_f32(np.array([0x3F80], np.uint16))[0] == 1.0


def test_f16_conversion_matches_numpy_everywhere():
    bits = np.arange(65536, dtype=np.uint16)
    f = oracle.f16_bits_to_f32(bits)
    ref = bits.view(np.float16).astype(np.float32)
    assert np.array_equal(f.view(np.uint32)[~np.isnan(ref)], ref.view(np.uint32)[~np.isnan(ref)])
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 200000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 2.0 ** -25, 2.0 ** -24, 5.96e-8, 6.1e-5,
                  np.inf, -np.inf], np.float32),
        # exact ties between adjacent halves
        (bits[:0x7bff].view(np.float16).astype(np.float32) + bits[1:0x7c00].view(np.float16).astype(np.float32)) / 2,
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.f32_to_f16_bits(x), x.astype(np.float16).view(np.uint16))


def test_bf16_round_to_nearest_even():
    # 1 + 2^-8 is an exact tie between 0x3F80 and 0x3F81 -> even; 1 + 3*2^-8 ties up to 0x3F82
    x = np.array([1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, 1.0 + 2.0 ** -8 + 2.0 ** -20], np.float32)
    assert oracle.f32_to_bf16(x).tolist() == [0x3F80, 0x3F82, 0x3F81]


def test_matmul_golden_exact(golden_dir):
    g = _load(golden_dir, "matmul_add_leakyrelu")
    out = oracle.matmul_bias_leakyrelu_f16_f32(g["input_a"], g["input_b"], g["input_bias"], 0.001)
    # integer-valued inputs: every product and partial sum is exact in f32
    assert np.max(np.abs(out - g["output"])) <= 1e-6 * np.max(np.abs(g["output"]))
    fails, mx, _ = oracle.compare(out, g["output"], atol=1.0, rtol=1e-2)
    assert fails == 0
    pos = g["output"] >= 0
    assert np.array_equal(out[pos], g["output"][pos])  # positives are untouched by the epilogue: bit-exact


def test_gather_golden_exact(golden_dir):
    g = _load(golden_dir, "gather_elementwise_fusion")
    out = oracle.relu_gather_cols_bias_f16(g["input_data"], g["input_indices"], g["input_bias"])
    # one f16 add after an exact relu: f32-then-round equals per-op f16 rounding
    assert np.array_equal(out.view(np.uint16), g["output_out"].view(np.uint16))


def test_transpose_golden_exact(golden_dir):
    g = _load(golden_dir, "relu_broadcast_transpose")
    out = oracle.relu_bcast_transpose_add_f16(g["input_data0"], g["input_data1"])
    assert np.array_equal(out.view(np.uint16), g["output_expected"].view(np.uint16))


def test_concat_golden_exact(golden_dir):
    g = _load(golden_dir, "add_broadcast_concat")
    out = oracle.add_mul_concat_f16(g["input_a"], g["input_b"], g["input_c"], g["input_d"])
    assert np.array_equal(out.view(np.uint16), g["output"].view(np.uint16))


def test_split_golden_within_reference_tolerance(golden_dir):
    g = _load(golden_dir, "split_relu_brc_add_mul")
    out = oracle.split_rows_relu_bias_scale_f16(g["input_a"], g["bias0"], g["bias1"], g["scale0"], g["scale1"])
    fails, mx, _ = oracle.compare(out.astype(np.float32), g["output"].astype(np.float32), atol=1e-2, rtol=1e-2)
    assert fails == 0
    # per-op f16 rounding vs the golden's single rounding differ by at most ~1.5 ulp of the result
    assert mx <= 2e-3


def test_reduce_golden_within_reference_tolerance(golden_dir):
    g = _load(golden_dir, "broadcast_add_reduce")
    out = oracle.bcast_add_rowsum_f16(g["input_a"], g["input_b"])
    fails, mx, _ = oracle.compare(out.astype(np.float32), g["output_c"].astype(np.float32), atol=10.0, rtol=1e-2)
    assert fails == 0
    assert mx <= 0.5  # 512 f16-rounded addends, |sum| up to ~500


def test_rowsum_f32_orderings_within_bound():
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, 64).astype(np.float32)
    b = rng.uniform(-1, 1, (64, 4096)).astype(np.float32)
    out, s64, abs64 = oracle.bcast_add_rowsum_f32(a, b, with_bounds=True)
    assert np.array_equal(out, oracle.bcast_add_rowsum_f32(a, b))
    assert np.all(np.abs(out - s64) <= 1e-5 * abs64)


def test_add_mul_f32_no_contraction():
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, 100003).astype(np.float32)
    b = rng.uniform(-1, 1, 100003).astype(np.float32)
    out = oracle.add_mul_f32(a, b)
    assert np.array_equal(out, (a + b) * b)  # numpy rounds after each op too
    fused = ((a.astype(np.float64) + b.astype(np.float64)) * b.astype(np.float64)).astype(np.float32)
    assert np.any(out != fused)  # the two-rounding result is distinguishable from a single rounding


def test_gather_rows_matches_numpy_restatement():
    rng = np.random.default_rng(0)
    table = oracle.f32_to_bf16(rng.standard_normal((1000, 64)).astype(np.float32))
    idx = rng.integers(0, 1000, 300).astype(np.int32)
    idx[:10] = idx[10:20]  # duplicates
    scale = oracle.f32_to_bf16(rng.uniform(0.5, 1.5, 64).astype(np.float32))
    resid = oracle.f32_to_bf16(rng.standard_normal((300, 64)).astype(np.float32))
    out = oracle.gather_rows_scale_resid_bf16(table, idx, scale, resid)
    t = oracle.bf16_to_f32(table)[idx]
    prod = oracle.bf16_to_f32(oracle.f32_to_bf16(t * oracle.bf16_to_f32(scale)[None, :]))
    want = oracle.f32_to_bf16(prod + oracle.bf16_to_f32(resid))
    assert np.array_equal(out, want)
    with pytest.raises(IndexError):
        bad = idx.copy()
        bad[5] = 1000
        oracle.gather_rows_scale_resid_bf16(table, bad, scale, resid)


def test_matmul_bf16_matches_f64_sample():
    rng = np.random.default_rng(0)
    M, K, N = 64, 512, 96
    A = oracle.f32_to_bf16((rng.standard_normal((M, K)) * 0.02).astype(np.float32))
    B = oracle.f32_to_bf16((rng.standard_normal((K, N)) * 0.02).astype(np.float32))
    bias = oracle.f32_to_bf16((rng.standard_normal(N) * 0.1).astype(np.float32))
    out = oracle.bf16_to_f32(oracle.matmul_bias_leakyrelu_bf16(A, B, bias, 0.01))
    x = oracle.bf16_to_f32(A).astype(np.float64) @ oracle.bf16_to_f32(B).astype(np.float64) + oracle.bf16_to_f32(bias)
    want = np.maximum(x, 0.01 * x)
    assert np.all(np.abs(out - want) <= 1e-2 * np.abs(want) + 1e-6)
    assert abs(oracle.matmul_bias_leakyrelu_bf16_at(A, B, bias, 0.01, 3, 5) - want[3, 5]) < 1e-9


def test_split_cfg_form_bias_axes():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 8, 32)).astype(np.float16)
    bias = (rng.standard_normal(8) * 0.1).astype(np.float16)
    out = oracle.split_relu_bias_mul_f16(x, bias, bias_axis=1)
    h0, h1 = x[..., :16], x[..., 16:]
    t = np.maximum(h0, np.float16(0))
    t = (t + bias[None, :, None]).astype(np.float16)
    want = (t * h1).astype(np.float16)
    assert np.array_equal(out.view(np.uint16), want.view(np.uint16))
    bias2 = (rng.standard_normal(16) * 0.1).astype(np.float16)
    out2 = oracle.split_relu_bias_mul_f16(x, bias2, bias_axis=2)
    t2 = (np.maximum(h0, np.float16(0)) + bias2[None, None, :]).astype(np.float16)
    assert np.array_equal(out2.view(np.uint16), (t2 * h1).astype(np.float16).view(np.uint16))
