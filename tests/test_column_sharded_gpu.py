"""Two GPUs, the reduced axis sharded: every rank runs the row-reduction kernel on its column slice through the
C-ABI, then one NCCL all-reduce of the f32 partial sums; and the same with the exchange inside the kernel
(partial sums stored into the peers' mailboxes over NVLink, no library collective).  Skipped on boxes with a
single GPU."""
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


EXCHANGE_SCRIPT = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["AFIR_ROOT"])
from ascend_mlir_b200 import configs, descriptors, sharding
from ascend_mlir_b200.runtime import CudaRuntime
from oracle import oracle
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
rt = CudaRuntime(); rt.set_device(local)
spec = descriptors.bcast_add_rowsum("f32")
x = sharding.RowsumExchange(local, rank, world, max_rows=4096)
x.connect()
dist.barrier()
outs, wants = [], []
# five calls back to back without a host synchronisation between them: both mailbox halves are reused while the
# other rank may be a call ahead; two shapes so that the staged and the plain kernel both send
for call, (M, N) in enumerate([(2048, 8192), (2048, 8192), (300, 1000), (4096, 4096), (2048, 8192)]):
    full = configs.broadcast_add_reduce(M=M, N=N, seed=20 + call)
    b, xs = full.inputs
    lo, hi = sharding.col_range(N, rank, world, quantum=4)
    b_d, x_d = torch.from_numpy(b).cuda(), torch.from_numpy(xs).cuda()   # the whole matrix resident, the slice is a view
    out = torch.full((M,), float("nan"), device="cuda")
    x.bcast_add_rowsum(b_d.data_ptr(), x_d.data_ptr() + lo * 4, out.data_ptr(), M, hi - lo, N)
    outs.append(out)
    wants.append((b, xs, lo, hi, b_d, x_d))
torch.cuda.synchronize()
x.check()
for out, (b, xs, lo, hi, b_d, x_d) in zip(outs, wants):
    M = b.shape[0]
    # every rank holds the same bits
    both = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(both, out)
    assert all(torch.equal(both[0], t) for t in both)
    # and they are the rank-ordered f32 sum of the partial sums the ordinary entry point produces
    mine = x_d[:, lo:hi].contiguous()
    partial = torch.empty(M, device="cuda")
    nb = lambda t: t.numel() * t.element_size()
    rt.launch_device(spec.binary, spec.name, [(b_d.data_ptr(), nb(b_d)), (mine.data_ptr(), nb(mine))],
                     [(partial.data_ptr(), nb(partial))], spec.pack({"M": M, "N": hi - lo}), 0, spec.magic)
    rt.synchronize()
    parts = [torch.empty_like(partial) for _ in range(world)]
    dist.all_gather(parts, partial)
    total = parts[0].clone()
    for t in parts[1:]:
        total += t
    assert torch.equal(out, total), float((out - total).abs().max())
    _, s64, abs64 = oracle.bcast_add_rowsum_f32(b, xs, with_bounds=True)
    assert np.all(np.abs(out.cpu().numpy() - s64) <= 1e-5 * abs64)
# the same through a compiled descriptor: afirt_executor_launch_device_exchange on this rank's contiguous slice
out2 = torch.full((M,), float("nan"), device="cuda")
rt.launch_device(spec.binary, spec.name, [(b_d.data_ptr(), nb(b_d)), (mine.data_ptr(), nb(mine))],
                 [(out2.data_ptr(), nb(out2))], spec.pack({"M": M, "N": hi - lo}), 0, spec.magic, exchange=x)
rt.synchronize()
x.check()
assert torch.equal(out2, total)
dist.barrier()
# a wait that runs out: rank 0 makes one more call, nobody answers; after 2 s the kernel gives up, the status
# says so and the context is still usable
if rank == 0:
    out = torch.full((2048,), float("nan"), device="cuda")
    x.bcast_add_rowsum(b_d.data_ptr(), x_d.data_ptr(), out.data_ptr(), 2048, 4096, 8192)
    torch.cuda.synchronize()
    try:
        x.check()
        raise SystemExit("the exchange did not report the missing rank")
    except RuntimeError as e:
        assert "gave up waiting" in str(e), str(e)
    assert bool(torch.isnan(out).all())             # no row was finished
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0  # the device still computes
    x.check()                                       # and the status was cleared by the report
dist.barrier()
x.close()
dist.destroy_process_group()
print(f"rank {rank} ok", flush=True)
'''


def _torchrun(script, tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = {**os.environ, "AFIR_ROOT": str(ROOT), "NCCL_NVLS_ENABLE": "0"}
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                           "127.0.0.1", "--master-port", str(port), str(script)], capture_output=True, text=True, env=env, timeout=600)


def test_exchange_inside_the_kernel_on_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank_exchange.py"
    script.write_text(EXCHANGE_SCRIPT)
    r = _torchrun(script, tmp_path)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


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
