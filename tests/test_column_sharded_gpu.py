"""Two GPUs, the reduced axis sharded: every rank runs the row-reduction kernel on its column slice through the
C-ABI, then one NCCL all-reduce of the f32 partial sums.  Skipped on boxes with a single GPU."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

RANK_SCRIPT = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["AFIR_ROOT"])
from ascend_mlir_b200 import configs, descriptors, sharding
from ascend_mlir_b200.runtime import CudaRuntime
from oracle import oracle
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
full = configs.broadcast_add_reduce(M=2048, N=4096, seed=9)
b, x = full.inputs
lo, hi = sharding.col_range(x.shape[1], rank, world, quantum=4)
mine = np.ascontiguousarray(x[:, lo:hi])
spec = descriptors.bcast_add_rowsum("f32")
rt = CudaRuntime(); rt.set_device(local)
partial = np.zeros(x.shape[0], np.float32)
rt.run(spec.binary, spec.name, [b, mine], [partial], spec.pack({"M": x.shape[0], "N": hi - lo}), 0, spec.magic)
total = sharding.allreduce_partial_rowsums(torch.from_numpy(partial).cuda()).cpu().numpy()
_, s64, abs64 = oracle.bcast_add_rowsum_f32(b, x, with_bounds=True)
assert np.all(np.abs(total - s64) <= 1e-5 * abs64), float(np.max(np.abs(total - s64) / abs64))
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok", flush=True)
'''


def test_column_sharded_reduction_on_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = {**os.environ, "AFIR_ROOT": str(ROOT), "NCCL_NVLS_ENABLE": "0"}
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
