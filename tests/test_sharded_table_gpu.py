"""Row gather from a table given as row shards (afirt_executor_launch_device_sharded_table).  On one GPU the shards are
separate buffers of the same device, which exercises the kernel and the launch path bit for bit; with two GPUs
every rank keeps one shard and reads the other through CUDA IPC over NVLink (afirt_peer_*)."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from ascend_mlir_b200 import configs
from ascend_mlir_b200.runtime.executor import CudaRuntime, ExecutorError
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _launch(torch, rt, w, table_shards, rows_per_shard, idx=None):
    table, idx0, scale, resid = w.inputs
    idx = idx0 if idx is None else idx
    dev = [torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (idx, scale, resid)]
    out = torch.zeros(w.out_shape, dtype=torch.uint16, device="cuda")
    nb = lambda t: t.numel() * t.element_size()
    inputs = [(table_shards[0], table.nbytes)] + [(t.data_ptr(), nb(t)) for t in dev]
    rt.launch_device(w.spec.binary, w.spec.name, inputs, [(out.data_ptr(), nb(out))], w.spec.pack(w.shape), 0, w.spec.magic,
                     table_shards=table_shards, rows_per_shard=rows_per_shard)
    rt.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("table_rows,rows_per_shard,width", [(4096, 2048, 256), (5000, 1250, 64), (1000, 400, 24), (777, 1024, 8)])
def test_shards_on_one_device_match_the_single_table(table_rows, rows_per_shard, width):
    import torch
    rt = CudaRuntime()
    rt.set_device(0)
    w = configs.gather_elementwise(table_rows, width, rows=3001, seed=table_rows)
    table = w.inputs[0]
    shards = [torch.from_numpy(np.ascontiguousarray(table[b:b + rows_per_shard])).cuda() for b in range(0, table_rows, rows_per_shard)]
    got = _launch(torch, rt, w, [s.data_ptr() for s in shards], rows_per_shard)
    want = oracle.gather_rows_scale_resid_bf16(*w.inputs)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_sharded_table_argument_errors():
    import torch
    rt = CudaRuntime()
    rt.set_device(0)
    w = configs.gather_elementwise(1024, 64, rows=100, seed=1)
    shard = torch.from_numpy(np.ascontiguousarray(w.inputs[0][:512])).cuda()
    with pytest.raises(ExecutorError, match="do not cover"):
        _launch(torch, rt, w, [shard.data_ptr()], 512)
    with pytest.raises(ExecutorError, match="rows_per_shard"):
        _launch(torch, rt, w, [shard.data_ptr(), shard.data_ptr()], 0)
    from ascend_mlir_b200 import descriptors
    ew = descriptors.add_mul("f32")
    m = torch.zeros(8, 8, device="cuda")
    with pytest.raises(ExecutorError, match="only a single gather group"):
        rt.launch_device(ew.binary, ew.name, [(m.data_ptr(), 256), (m.data_ptr(), 256)], [(m.data_ptr(), 256)],
                         ew.pack({"M": 8, "N": 8}), 0, ew.magic, table_shards=[m.data_ptr()], rows_per_shard=8)
    # an index past the table is counted and reported, as with a single table
    bad = w.inputs[1].copy()
    bad[7] = 5000
    with pytest.raises(ExecutorError, match="out of range|index"):
        _launch(torch, rt, w, [shard.data_ptr(), shard.data_ptr()], 512, idx=bad)


RANK_SCRIPT = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["AFIR_ROOT"])
from ascend_mlir_b200 import configs, sharding
from ascend_mlir_b200.runtime import CudaRuntime
from oracle import oracle
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
rt = CudaRuntime(); rt.set_device(local)
T, W = 8192, 256
full = configs.gather_elementwise(T, W, rows=20000, seed=77)      # the same table and indices on every rank (same seed)
w = full.shard(rank, world)                                      # output rows (indices, resid) are row-sharded as always
table = full.inputs[0]
R = T // world
filler = torch.empty(12345, dtype=torch.uint8, device="cuda")    # so that the shard sits INSIDE a block of the caching allocator
mine = torch.from_numpy(np.ascontiguousarray(table[rank * R:(rank + 1) * R])).cuda()
st = sharding.ShardedTable(mine, local, R)
dist.barrier()
_, idx, scale, resid = w.inputs
dev = [torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (idx, scale, resid)]
out = torch.zeros(w.out_shape, dtype=torch.uint16, device="cuda")
nb = lambda t: t.numel() * t.element_size()
for _ in range(2):
    rt.launch_device(w.spec.binary, w.spec.name, [(st.pointers[0], table.nbytes)] + [(t.data_ptr(), nb(t)) for t in dev],
                     [(out.data_ptr(), nb(out))], w.spec.pack(w.shape), 0, w.spec.magic, table_shards=st.pointers, rows_per_shard=R)
rt.synchronize()
want = oracle.gather_rows_scale_resid_bf16(table, idx, scale, resid)
assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
remote = int(((idx // R) != rank).sum())
assert remote > 0
dist.barrier()
st.close()
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok, {remote} of {idx.shape[0]} rows came from the other GPU", flush=True)
'''


def test_table_sharded_over_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank_table.py"
    script.write_text(RANK_SCRIPT)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = {**os.environ, "AFIR_ROOT": str(ROOT), "NCCL_NVLS_ENABLE": "0"}
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
