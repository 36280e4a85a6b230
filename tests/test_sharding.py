"""Row sharding of the fused groups (no collective on the data path) and the cross-rank bookkeeping,
exercised with world_size-2 gloo ranks on CPU."""
import os
import socket

import numpy as np
import pytest

from ascend_mlir_b200 import configs
from ascend_mlir_b200.configs import row_range
from oracle import oracle


@pytest.mark.parametrize("total,world", [(8192, 8), (10, 4), (3, 8), (0, 2), (32, 1), (262144, 3)])
def test_row_range_is_a_balanced_contiguous_partition(total, world):
    ranges = [row_range(total, r, world) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == total
    for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
        assert a1 == b0
    sizes = [b - a for a, b in ranges]
    assert max(sizes) - min(sizes) <= 1


def _oracle_out(w):
    n = w.name
    if n == "elementwise_chain":
        return oracle.add_mul_f32(*w.inputs)
    if n == "split_relu_broadcast_add_mul":
        return oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], 1).view(np.uint16)
    if n == "broadcast_add_reduce":
        return oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1])
    if n == "gather_elementwise":
        return oracle.gather_rows_scale_resid_bf16(*w.inputs)
    return oracle.matmul_bias_leakyrelu_bf16(*w.inputs, 0.01)


SMALL = {
    "elementwise_chain": dict(M=37, N=64),
    "split_relu_broadcast_add_mul": dict(B=5, R=16, C=32),
    "broadcast_add_reduce": dict(M=29, N=128),
    "gather_elementwise": dict(table_rows=200, width=32, rows=45),
    "matmul_add_leakyrelu": dict(M=21, N=32, K=40),
}


@pytest.mark.parametrize("name", list(SMALL))
@pytest.mark.parametrize("world", [2, 4, 8])
def test_shards_reassemble_to_the_unsharded_result(name, world):
    full = configs.CONFIGS[name](**SMALL[name])
    want = _oracle_out(full)
    parts = []
    units = 0
    for r in range(world):
        s = full.shard(r, world)
        units += s.units
        assert s.spec is full.spec  # same kernel binary on every rank; only TilingData dims differ
        parts.append(_oracle_out(s).reshape((s.units,) + want.shape[1:]))
    assert units == full.units
    assert np.array_equal(np.concatenate(parts, axis=0), want)


@pytest.mark.parametrize("world", [2, 3, 8])
def test_transposed_operand_shards_by_columns_of_the_transposed_input(world):
    """out[n, m] = (a[m, n] + b[n, m]) * c[n] sharded by output rows: a rank owns columns of `a`, rows of `b`, a piece
    of `c`; the shards' results stack to the unsharded one and the tiling dims of a shard are (M, its rows)."""
    full = configs.transposed_add_mul(M=24, N=37)
    want = full.expected()
    parts, units = [], 0
    for r in range(world):
        s = full.shard(r, world)
        units += s.units
        assert s.spec is full.spec and s.shape == {"M": 24, "N": s.units}
        assert s.inputs[0].shape == (24, s.units) and s.inputs[0].flags["C_CONTIGUOUS"] and s.out_shape == (s.units, 24)
        parts.append(s.expected())
    assert units == full.units == 37
    assert np.array_equal(np.concatenate(parts, axis=0).view(np.uint16), want.view(np.uint16))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ascend_mlir_b200 import sharding
        full = configs.broadcast_add_reduce(M=30, N=64, seed=0)
        mine = full.shard(rank, world)
        out = oracle.bcast_add_rowsum_f32(mine.inputs[0], mine.inputs[1])
        # every rank reports its own fake step time; the job time is the slowest rank's
        rate, ms = sharding.job_throughput(mine.algorithmic_bytes, 1.0 + rank)
        assert sharding.world() == (rank, world)
        q.put((rank, out, rate, ms, mine.algorithmic_bytes))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_without_a_data_collective():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=120) for _ in procs), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    full = configs.broadcast_add_reduce(M=30, N=64, seed=0)
    want = oracle.bcast_add_rowsum_f32(full.inputs[0], full.inputs[1])
    assert np.array_equal(np.concatenate([g[1] for g in got]), want)
    total_bytes = sum(g[4] for g in got)
    for _, _, rate, ms, _ in got:
        assert ms == 2.0  # max over ranks of (1.0, 2.0)
        assert rate == pytest.approx(total_bytes / 2e-3)


# ---- the reduced axis sharded: partial row sums + one all-reduce ---------------------------------------------------
def _column_rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ascend_mlir_b200 import sharding
        full = configs.broadcast_add_reduce(M=37, N=100, seed=5)
        b, x = full.inputs
        lo, hi = sharding.col_range(x.shape[1], rank, world, quantum=4)
        # the row-broadcast operand counts once per column of the slice, exactly as in the unsharded sum
        partial = oracle.bcast_add_rowsum_f32(b, np.ascontiguousarray(x[:, lo:hi]))
        total = sharding.allreduce_partial_rowsums(torch.from_numpy(partial.copy()))
        q.put((rank, (lo, hi), total.numpy()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_col_range_partitions_in_vector_units():
    from ascend_mlir_b200 import sharding
    for total, world, quantum in [(100, 2, 4), (8192, 8, 4), (10, 4, 4), (7, 3, 1)]:
        pieces = [sharding.col_range(total, r, world, quantum) for r in range(world)]
        assert pieces[0][0] == 0 and pieces[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
        assert all(lo % quantum == 0 or lo == total for lo, _ in pieces)


def test_two_gloo_ranks_column_sharded_reduction_needs_one_allreduce():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_column_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=120) for _ in procs), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0][1] == (0, 52) and got[1][1] == (52, 100)
    full = configs.broadcast_add_reduce(M=37, N=100, seed=5)
    _, s64, abs64 = oracle.bcast_add_rowsum_f32(full.inputs[0], full.inputs[1], with_bounds=True)
    for _, _, total in got:
        assert np.array_equal(total, got[0][2]), "every rank ends with the same sums"
        assert np.all(np.abs(total - s64) <= 1e-5 * abs64)
