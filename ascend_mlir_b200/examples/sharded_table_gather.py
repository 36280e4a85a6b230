#!/usr/bin/env python3
"""gather_elementwise with the TABLE sharded by rows over the GPUs of one node, timed against the replicated table:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29517 \
        -m ascend_mlir_b200.examples.sharded_table_gather [--table-rows 1048576] [--width 256] [--rows 262144]

Every rank gathers `rows` output rows (its own indices, scale and residual, as in the row-sharded benchmark) from a
bf16 table of `table-rows` x `width`:
  replicated   the whole table in every GPU's memory (the benchmark's layout: 512 MiB per GPU at the defaults)
  sharded      rank r keeps rows [r * T / N, (r + 1) * T / N) only; the kernel reads the other ranks' rows straight
               from their memory over NVLink (CUDA IPC mappings, plain loads): 1 / N of the table per GPU, no exchange
               step, no library collective
Both results are compared bit for bit before timing.  Time is CUDA events over `steps` calls, MAX over ranks; rank 0
prints one JSON line.  NVLink moves (N - 1) / N of the gathered bytes in the sharded layout, so it is bound by the
link (about 770 GB/s per direction per GPU measured on this kind of box), not by HBM.
"""
import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from ascend_mlir_b200 import descriptors, sharding
from ascend_mlir_b200.runtime import CudaRuntime


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--table-rows", type=int, default=1048576)
    ap.add_argument("--width", type=int, default=256)
    ap.add_argument("--rows", type=int, default=262144)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rt = CudaRuntime()
    rt.set_device(local)
    spec = descriptors.gather_rows_scale_resid("bf16", "i32")
    T, W, R = args.table_rows, args.width, args.rows
    per = (T + world - 1) // world
    g = torch.Generator(device="cuda").manual_seed(7)               # the same table on every rank
    table = torch.randn(T, W, device="cuda", generator=g).to(torch.bfloat16)
    mine = table[rank * per:min(T, (rank + 1) * per)].clone()
    gi = torch.Generator(device="cuda").manual_seed(100 + rank)     # every rank's own indices and residual
    idx = torch.randint(0, T, (R,), device="cuda", generator=gi, dtype=torch.int32)
    scale = (torch.rand(W, device="cuda", generator=gi) + 0.5).to(torch.bfloat16)
    resid = torch.randn(R, W, device="cuda", generator=gi).to(torch.bfloat16)
    out_a = torch.zeros(R, W, device="cuda", dtype=torch.bfloat16)
    out_b = torch.zeros_like(out_a)
    st = sharding.ShardedTable(mine, local, per)
    dist.barrier()
    nb = lambda t: t.numel() * t.element_size()
    tiling = spec.pack({"T": T, "W": W, "R": R})
    stream = torch.cuda.current_stream().cuda_stream
    tail = [(idx.data_ptr(), nb(idx)), (scale.data_ptr(), nb(scale)), (resid.data_ptr(), nb(resid))]

    def replicated():
        rt.launch_device(spec.binary, spec.name, [(table.data_ptr(), nb(table))] + tail, [(out_a.data_ptr(), nb(out_a))], tiling, 0,
                         spec.magic, stream=stream)

    def sharded():
        rt.launch_device(spec.binary, spec.name, [(st.pointers[0], nb(table))] + tail, [(out_b.data_ptr(), nb(out_b))], tiling, 0,
                         spec.magic, stream=stream, table_shards=st.pointers, rows_per_shard=per)

    replicated()
    sharded()
    rt.synchronize()
    torch.cuda.synchronize()
    same = bool(torch.equal(out_a.view(torch.int16), out_b.view(torch.int16)))
    micros = {}
    for name, fn in (("replicated", replicated), ("sharded", sharded)):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        micros[name] = round(sharding.max_over_ranks(e0.elapsed_time(e1) / args.steps, "cuda") * 1000, 1)
    rt.synchronize()
    if rank == 0:
        row_bytes = W * 2
        work = R * 4 + 3 * R * row_bytes + row_bytes     # indices, gathered rows, residual, output, scale (per rank)
        remote = R * row_bytes * (world - 1) / world     # gathered bytes that cross NVLink into each GPU (uniform indices)
        print(json.dumps({"example": "sharded_table_gather", "n_gpus": world, "table_rows": T, "width": W, "rows_per_rank": R,
                          "table_bytes_per_gpu": {"replicated": T * row_bytes, "sharded": per * row_bytes},
                          "microseconds_per_call": micros,
                          "whole_job_GBs": {k: round(world * work / (v * 1e-6) / 1e9, 1) for k, v in micros.items()},
                          "nvlink_inbound_GBs_per_gpu": round(remote / (micros["sharded"] * 1e-6) / 1e9, 1),
                          "sharded_equals_replicated_bits": same}), flush=True)
    dist.barrier()
    st.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0 if same else 1


if __name__ == "__main__":
    raise SystemExit(main())
