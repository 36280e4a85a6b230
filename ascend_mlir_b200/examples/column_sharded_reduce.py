#!/usr/bin/env python3
"""broadcast_add_reduce with the REDUCED axis sharded over the GPUs of one node, three ways, timed:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29517 \
        -m ascend_mlir_b200.examples.column_sharded_reduce [--rows 8192] [--cols 8192] [--steps 200]

  local_kernel_only            every rank reduces its column slice and stops (no exchange: the lower bound)
  kernel_plus_nccl_allreduce   the same kernel, then one NCCL all-reduce of the f32 partial sums
  fused_exchange               one kernel per rank that also exchanges the partial sums through peer-mapped
                               mailboxes (afirt_rowsum_exchange_* of the C-ABI library)

Every rank holds the whole matrix in its memory and reads its column slice in place (row stride = cols), inputs
rotate over three buffer sets, time is CUDA events on the launching stream over `steps` back-to-back calls, MAX
over ranks.  The fused result is checked against the two-step result before timing (same f32 additions in rank
order: equal bits for two ranks).  Rank 0 prints one JSON line (microseconds per call and whole-job GB/s).
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from ascend_mlir_b200 import descriptors, sharding
from ascend_mlir_b200.runtime import CudaRuntime


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rt = CudaRuntime()
    rt.set_device(local)
    spec = descriptors.bcast_add_rowsum("f32")
    M, N = args.rows, args.cols
    lo, hi = sharding.col_range(N, rank, world, quantum=4)
    g = torch.Generator(device="cuda").manual_seed(1)  # the same matrix on every rank
    sets = [(torch.rand(M, device="cuda", generator=g) - 0.5, torch.rand(M, N, device="cuda", generator=g) - 0.5) for _ in range(3)]
    slices = [(a, b[:, lo:hi].contiguous()) for a, b in sets]
    out = torch.empty(M, device="cuda")
    exchange = sharding.RowsumExchange(local, rank, world, max_rows=M)
    exchange.connect()
    dist.barrier()
    nbytes = lambda t: t.numel() * t.element_size()
    stream = torch.cuda.current_stream().cuda_stream
    tiling = spec.pack({"M": M, "N": hi - lo})

    def local_only(i):
        a, mine = slices[i % 3]
        rt.launch_device(spec.binary, spec.name, [(a.data_ptr(), nbytes(a)), (mine.data_ptr(), nbytes(mine))],
                         [(out.data_ptr(), nbytes(out))], tiling, 0, spec.magic, stream=stream)

    def two_step(i):
        local_only(i)
        dist.all_reduce(out)

    def fused(i):
        a, b = sets[i % 3]
        exchange.bcast_add_rowsum(a.data_ptr(), b.data_ptr() + lo * 4, out.data_ptr(), M, hi - lo, N, "f32", stream)

    two_step(0)
    want = out.clone()
    fused(0)
    torch.cuda.synchronize()
    exchange.check()
    same_bits = bool(torch.equal(out, want))
    close = bool(torch.allclose(out, want, rtol=1e-5, atol=1e-3))

    micros = {}
    for name, fn in (("local_kernel_only", local_only), ("kernel_plus_nccl_allreduce", two_step), ("fused_exchange", fused)):
        for i in range(args.warmup):
            fn(i)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        micros[name] = round(sharding.max_over_ranks(e0.elapsed_time(e1) / args.steps, "cuda") * 1000, 2)
    exchange.check()
    if rank == 0:
        work = M * N * 4 + 2 * M * 4  # the matrix once, the broadcast operand and the result
        print(json.dumps({"example": "column_sharded_reduce", "n_gpus": world, "rows": M, "cols": N, "steps": args.steps,
                          "microseconds_per_call": micros,
                          "whole_job_GBs": {k: round(work / (v * 1e-6) / 1e9, 1) for k, v in micros.items()},
                          "fused_equals_two_step_bits": same_bits, "fused_close_to_two_step": close}), flush=True)
    dist.barrier()
    exchange.close()
    dist.destroy_process_group()
    return 0 if close else 1


if __name__ == "__main__":
    raise SystemExit(main())
