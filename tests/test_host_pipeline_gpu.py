"""Host-pointer runs large enough to be cut into leading-axis chunks (copies in, kernel and copies out of
successive chunks overlap) must give the same bytes as the single-shot path and match the oracle."""
import os

import numpy as np
import pytest

from ascend_mlir_b200 import configs, descriptors
from ascend_mlir_b200.runtime.executor import CudaRuntime
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    r = CudaRuntime()
    r.set_device(0)
    return r


def both_paths(rt, w, **tile):
    outs = []
    for no_pipe in ("", "1"):
        if no_pipe:
            os.environ["AFIR_CUDA_NO_PIPELINE"] = "1"
        else:
            os.environ.pop("AFIR_CUDA_NO_PIPELINE", None)
        try:
            out = w.new_output()
            rt.run(w.spec.binary, w.spec.name, w.inputs, [out], w.tiling(**tile), block_dim=0, magic=w.spec.magic)
            outs.append((out, rt.last_launch_count))
        finally:
            os.environ.pop("AFIR_CUDA_NO_PIPELINE", None)
    (piped, n_piped), (single, n_single) = outs
    assert n_piped > n_single >= 1, "the large run was expected to be chunked"
    return piped, single


def test_elementwise_chain_chunked(rt):
    w = configs.elementwise_chain(2051, 2048, seed=41)  # odd row count: ragged last chunk
    piped, single = both_paths(rt, w)
    assert np.array_equal(piped, single) and np.array_equal(piped, oracle.add_mul_f32(*w.inputs))


def test_split_group_chunked_views_of_one_argument(rt):
    w = configs.split_relu_broadcast_add_mul(67, 128, 512, seed=42)
    piped, single = both_paths(rt, w)
    want = oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], 1)
    assert np.array_equal(piped.view(np.uint16), single.view(np.uint16))
    assert np.array_equal(piped.view(np.uint16), want.view(np.uint16))


def test_row_reduce_chunked(rt):
    w = configs.broadcast_add_reduce(3000, 4096, seed=43)
    piped, single = both_paths(rt, w)
    _, s64, abs64 = oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1], with_bounds=True)
    for out in (piped, single):
        assert np.all(np.abs(out - s64) <= 1e-5 * abs64)


def test_gather_rows_chunked_and_bad_index_still_reported(rt):
    w = configs.gather_elementwise(30000, 256, 20011, seed=44)
    piped, single = both_paths(rt, w)
    assert np.array_equal(piped, single) and np.array_equal(piped, oracle.gather_rows_scale_resid_bf16(*w.inputs))
    w.inputs[1][20000] = 30000  # lands in the last chunk
    from ascend_mlir_b200.runtime import ExecutorError
    with pytest.raises(ExecutorError, match=r"gather index out of range \(1 indices\)"):
        rt.run(w.spec.binary, w.spec.name, w.inputs, [w.new_output()], w.tiling())


def test_matmul_chunked_rows(rt):
    w = configs.matmul_add_leakyrelu(3000, 1024, 2048, seed=45)
    piped, single = both_paths(rt, w)
    assert np.array_equal(piped, single)
    rows = slice(1400, 1600)  # straddles a chunk boundary
    want = oracle.bf16_to_f32(oracle.matmul_bias_leakyrelu_bf16(w.inputs[0][rows], w.inputs[1], w.inputs[2], 0.01))
    got = oracle.bf16_to_f32(piped[rows])
    assert np.all(np.abs(got - want) <= 1e-2 * np.abs(want) + 1e-3)
