"""Programmatic dependent launch keeps the stream's order.  Elementwise, reduction and transpose kernels are launched
with programmatic stream serialisation and wait for the previous kernel of the stream themselves (first thing, before
any global access).  A chain whose every kernel reads what the previous one wrote -- (a + b) * b, then its transpose,
then the row sums of the transpose -- is enqueued on one stream without any host synchronisation, directly and as a
replayed CUDA graph, over intermediates that were poisoned with NaN beforehand: a kernel that started before its
predecessor had finished would read the poison.  The same chain runs in a child process with AFIR_CUDA_PDL=0 (ordinary
launches) and must give the same bits."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHAIN = r'''
import sys
import numpy as np
sys.path.insert(0, sys.argv[1])
import torch
from ascend_mlir_b200 import descriptors
from ascend_mlir_b200.runtime.executor import CudaRuntime

M, N = 1536, 2048   # 12 MB per tensor: kernels of a few microseconds, so the launches really are back to back
rt = CudaRuntime(); rt.set_device(0)
ew, tr, rr = descriptors.add_mul("f32"), descriptors.transpose_2d("f32"), descriptors.bcast_add_rowsum("f32")
rng = np.random.default_rng(7)
a_h = rng.uniform(-1, 1, (M, N)).astype(np.float32)
b_h = rng.uniform(-1, 1, (M, N)).astype(np.float32)
bias_h = rng.uniform(-1, 1, N).astype(np.float32)
a, b, bias = (torch.from_numpy(x).cuda() for x in (a_h, b_h, bias_h))
c = torch.empty(M, N, device="cuda"); ct = torch.empty(N, M, device="cuda"); out = torch.empty(N, device="cuda")
nb = lambda t: t.numel() * t.element_size()
arg = lambda t: (t.data_ptr(), nb(t))
stream = torch.cuda.Stream()

def chain(s):
    rt.launch_device(ew.binary, ew.name, [arg(a), arg(b)], [arg(c)], ew.pack({"M": M, "N": N}), 0, ew.magic, stream=s)
    rt.launch_device(tr.binary, tr.name, [arg(c)], [arg(ct)], tr.pack({"R": M, "C": N}), 0, tr.magic, stream=s)
    rt.launch_device(rr.binary, rr.name, [arg(bias), arg(ct)], [arg(out)], rr.pack({"M": N, "N": M}), 0, rr.magic, stream=s)

def poison():
    for t in (c, ct, out):
        t.fill_(float("nan"))
    torch.cuda.synchronize()

results = []
poison()
for _ in range(5):          # five chains back to back: each kernel follows another kernel of this library
    chain(stream.cuda_stream)
stream.synchronize()
results.append(out.cpu().numpy().copy())
graph = torch.cuda.CUDAGraph()
with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
    for _ in range(3):
        chain(torch.cuda.current_stream().cuda_stream)
for _ in range(2):
    poison()
    with torch.cuda.stream(stream):
        graph.replay()
    stream.synchronize()
    results.append(out.cpu().numpy().copy())
cth = ((a_h + b_h) * b_h).T
want = (bias_h[:, None].astype(np.float64) + cth.astype(np.float64)).sum(axis=1)
bound = 1e-5 * (np.abs(bias_h[:, None].astype(np.float64)) + np.abs(cth.astype(np.float64))).sum(axis=1)
for r in results:
    assert not np.isnan(r).any(), "a kernel read its predecessor's output before it was written"
    assert np.all(np.abs(r - want) <= bound)
    assert r.tobytes() == results[0].tobytes()
assert torch.equal(ct, c.t().contiguous())
sys.stdout.buffer.write(results[0].tobytes())
'''


def run_chain(pdl):
    env = dict(os.environ)
    env.pop("AFIR_CUDA_PDL", None)
    if pdl is not None:
        env["AFIR_CUDA_PDL"] = pdl
    r = subprocess.run([sys.executable, "-c", CHAIN, str(ROOT)], capture_output=True, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr.decode()[-3000:]
    return r.stdout


def test_dependent_kernels_keep_stream_order_and_match_ordinary_launches():
    with_attribute = run_chain(None)
    ordinary = run_chain("0")
    assert len(with_attribute) == 2048 * 4
    assert with_attribute == ordinary
