#!/usr/bin/env python3
"""Benchmark of the fused-group hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of one fused group over one batch of seeded synthetic input.  The default
workload is the split-relu-broadcast-add-mul group (f16 [32,1024,2048] -> [32,1024,1024]); the other
four benchmark groups and two transpose-class groups (a plain 2-D transpose and the reference's
relu-broadcast-transpose example at [8192,8192]) are timed the same way and reported under "groups".
`value` is device-resident throughput (CUDA events on the launching stream), `e2e` the same pass
through afirt_executor_run with pinned HOST buffers (H2D + kernel + D2H inside the timed region).
With N > 1 (torchrun, one rank per GPU) every rank runs a full-size batch of its own (the leading
axis grows with N and is sharded row-wise, no collective); the time is the max over ranks.
`--impl reference` times the CPU restatement of the reference semantics on the host cores instead.
"""
import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from ascend_mlir_b200 import configs  # noqa: E402

METRIC = "fused_group_hbm_throughput"
DEFAULT_WORKLOAD = "split_relu_broadcast_add_mul"
NOMINAL_HBM_GBS = 8000.0
NOMINAL_BF16_TFLOPS = 2250.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of each group's kernel at the bench
# shapes, from the ncu captures summarised in profiles/<kernel>__<workload>.md (measured once,
# not re-measured by this script: a profiler never runs inside a timed bench).
NCU_DRAM_BYTES_PER_LAUNCH = {
    "elementwise_chain": 158998016,
    "split_relu_broadcast_add_mul": 163837696,
    "broadcast_add_reduce": 271949824,
    "gather_elementwise": 363983360,
    "matmul_add_leakyrelu": 951392256,
    "transpose_2d": 217530624,
}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---- clocks ---------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while a region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.sm_max = [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    _NAMES = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
              0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
              0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._halt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self._NAMES.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def finish(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.sm_max,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- CPU reference arm ---------------------------------------------------------------------------------
def cpu_sample(name: str):
    """A bounded sample of the workload for the host-CPU leg: (workload, callable, description)."""
    from oracle import oracle
    if name == "elementwise_chain":
        w = configs.elementwise_chain()
        return w, (lambda: oracle.add_mul_f32(*w.inputs)), "full config, f32 [4096,4096]"
    if name == "split_relu_broadcast_add_mul":
        w = configs.split_relu_broadcast_add_mul()
        return w, (lambda: oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], 1)), "full config, f16 [32,1024,2048]"
    if name == "broadcast_add_reduce":
        w = configs.broadcast_add_reduce()
        return w, (lambda: oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1])), "full config, f32 [8192,8192]"
    if name == "gather_elementwise":
        w = configs.gather_elementwise()
        return w, (lambda: oracle.gather_rows_scale_resid_bf16(*w.inputs)), "full config, 262144 rows of a 1M-row table"
    if name == "matmul_add_leakyrelu":
        w = configs.matmul_add_leakyrelu(M=256)
        return w, (lambda: oracle.matmul_bias_leakyrelu_bf16(*w.inputs, 0.01)), "256 of 8192 output rows (N=K=8192)"
    if name == "transpose_2d":
        w = configs.transpose_2d()
        return w, (lambda: oracle.transpose_2d(w.inputs[0])), "full size, f16 [8192,8192]"
    if name == "relu_broadcast_transpose_add":
        w = configs.relu_broadcast_transpose_add()
        return w, (lambda: oracle.relu_bcast_transpose_add_f16(*w.inputs)), "full size, f16 [8192,8192]"
    raise SystemExit(f"unknown workload {name}")


def work_of(w):
    return (w.flops, "TFLOP/s", 1e12) if w.bound == "tensor" else (w.algorithmic_bytes, "GB/s", 1e9)


def time_cpu(name: str, steps: int, warmup: int):
    # torchrun exports OMP_NUM_THREADS=1; the CPU leg is meant to use every host core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from oracle import oracle
    oracle.set_num_threads(os.cpu_count() or 1)
    w, fn, sample = cpu_sample(name)
    for _ in range(max(1, min(warmup, 1))):
        fn()
    times = []
    budget = time.time() + 60.0
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
        if time.time() > budget:
            break
    work, unit, scale = work_of(w)
    best = min(times)
    return {"value": work / best / scale, "unit": unit, "cores": oracle.num_threads(), "kind": "port",
            "sample": sample, "seconds_per_pass": best, "passes": len(times)}, w


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu, w = time_cpu(args.workload, min(args.steps, 5), args.warmup)
    line = {"metric": METRIC, "value": cpu["value"], "unit": cpu["unit"], "n_gpus": args.gpus, "steps": cpu["passes"],
            "warmup": 1, "ms_per_step": cpu["seconds_per_pass"] * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype_of(args.workload), "data": "synthetic", "impl": "reference",
            "config": {"workload": args.workload, "note": "CPU restatement of the reference semantics (the reference's own "
                       "device path needs MLIR + CANN and cannot be built here), OpenMP over all host cores"},
            "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cpu["value"], "unit": cpu["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def dtype_of(name):
    return {"elementwise_chain": "f32", "split_relu_broadcast_add_mul": "f16", "broadcast_add_reduce": "f32",
            "gather_elementwise": "bf16", "matmul_add_leakyrelu": "bf16", "transpose_2d": "f16",
            "relu_broadcast_transpose_add": "f16"}[name]


# ---- GPU arm ------------------------------------------------------------------------------------------------
class DeviceGroup:
    """One workload resident on the device, launched through the C-ABI device entry point."""

    def __init__(self, torch, rt, w, device, stream, buffer_sets=3):
        self.torch, self.rt, self.w, self.stream = torch, rt, w, stream
        self.host_in = [torch.from_numpy(np.ascontiguousarray(x).view(np.int16) if x.dtype == np.uint16 else
                                         np.ascontiguousarray(x).view(np.int16) if x.dtype == np.float16 else
                                         np.ascontiguousarray(x)).pin_memory() for x in w.inputs]
        # Several identical sets of device buffers, used in rotation: a step then touches memory that was last used
        # `buffer_sets` steps earlier, so nothing of it is still in the 126 MB L2 (with one set, part of the previous
        # step's output would still be dirty in L2 and the figure would read above what HBM delivers).
        out_np_dtype = np.int16 if w.out_dtype.itemsize == 2 else w.out_dtype
        out_dtype = torch.from_numpy(np.zeros(1, out_np_dtype)).dtype
        self.sets = []
        for _ in range(max(1, buffer_sets)):
            ins = [t.to(device, non_blocking=False) for t in self.host_in]
            out = torch.empty(tuple(w.out_shape), dtype=out_dtype, device=device)
            self.sets.append((ins, out, [(t.data_ptr(), t.numel() * t.element_size()) for t in ins],
                              [(out.data_ptr(), out.numel() * out.element_size())]))
        self.dev_in, self.dev_out = self.sets[0][0], self.sets[0][1]
        self.host_out = torch.empty(tuple(w.out_shape), dtype=self.dev_out.dtype).pin_memory()
        self.turn = 0
        self.tiling = w.tiling()
        ws_bytes = rt.workspace_bytes(w.spec.binary, self.tiling)
        self.ws = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=device)
        self.host_in_args = [(t.data_ptr(), t.numel() * t.element_size()) for t in self.host_in]
        self.host_out_args = [(self.host_out.data_ptr(), self.host_out.numel() * self.host_out.element_size())]

    def launch(self, cuda_stream=None):
        _, _, in_args, out_args = self.sets[self.turn % len(self.sets)]
        self.turn += 1
        self.rt.launch_device(self.w.spec.binary, self.w.spec.name, in_args, out_args, self.tiling, 0, self.w.spec.magic,
                              (self.ws.data_ptr(), self.ws.numel()),
                              self.stream.cuda_stream if cuda_stream is None else cuda_stream)

    def run_host(self):
        self.rt.run_raw(self.w.spec.binary, self.w.spec.name, self.host_in_args, self.host_out_args, self.tiling, 0,
                        self.w.spec.magic)

    def timed(self, steps, warmup, sync, use_graph=True):
        """Milliseconds per step, kernels launched, and how they were launched.  The K launches of the timed
        region are captured once into a CUDA graph and replayed with a single graph launch, so the figure is
        device time of K back-to-back kernels whatever K is; if capture is refused the launches are issued
        one by one through the C-ABI as in the warm-up."""
        torch = self.torch
        for _ in range(warmup):
            self.launch()
        sync()
        graph, mode = None, "direct"
        if use_graph:
            try:
                before = self.rt.total_launch_count
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream, capture_error_mode="thread_local"):
                    for _ in range(steps):
                        self.launch(torch.cuda.current_stream().cuda_stream)
                launches = self.rt.total_launch_count - before
                with torch.cuda.stream(self.stream):
                    g.replay()  # one untimed replay: graph upload and first-use costs stay out of the timing
                sync()
                graph, mode = g, "cuda_graph"
            except Exception as e:  # capture refused: fall back to direct launches, and say so
                graph, mode = None, f"direct (graph capture failed: {type(e).__name__})"
                sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if graph is not None:
            with torch.cuda.stream(self.stream):
                e0.record(self.stream)
                graph.replay()
                e1.record(self.stream)
        else:
            before = self.rt.total_launch_count
            e0.record(self.stream)
            for _ in range(steps):
                self.launch()
            e1.record(self.stream)
            launches = self.rt.total_launch_count - before
        sync()
        self.rt.synchronize(self.stream.cuda_stream)
        self.launch_mode = mode
        return e0.elapsed_time(e1) / steps, launches

    def timed_e2e(self, steps, warmup, sync):
        for _ in range(warmup):
            self.run_host()
        sync()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.run_host()
        sync()
        return (time.perf_counter() - t0) * 1e3 / steps


def column_sharded_reduce(torch, dist, rt, device, stream, rank, world, local, steps=200, warmup=10):
    """The one exchange step the path has: broadcast_add_reduce with its REDUCED axis sharded (strong scaling,
    one 8192 x 8192 f32 matrix, every rank reads its column slice in place).  Times the slice kernel alone, the
    slice kernel followed by an NCCL all-reduce of the partial sums, and the kernel that exchanges the partial
    sums itself through peer-mapped mailboxes.  Every step that can fail on one rank only is followed by a MIN
    over ranks, so either all ranks go on or all stop; the waits inside the kernel are bounded."""
    from ascend_mlir_b200 import descriptors, sharding

    def all_ok(flag):
        t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    M, N = 8192, 8192
    spec = descriptors.bcast_add_rowsum("f32")
    lo, hi = sharding.col_range(N, rank, world, quantum=4)
    exchange, error = None, None
    try:
        exchange = sharding.RowsumExchange(local, rank, world, max_rows=M)
    except Exception as e:
        error = f"{type(e).__name__}: {e}"
    if not all_ok(exchange is not None):
        if exchange is not None:
            exchange.close()
        return {"error": error or "another rank could not create its mailbox"}
    try:
        exchange.connect()
    except Exception as e:
        error = f"{type(e).__name__}: {e}"
    if not all_ok(error is None):
        exchange.close()
        return {"error": error or "another rank could not map the mailboxes"}
    try:
        with torch.cuda.stream(stream):
            g = torch.Generator(device=device).manual_seed(1)  # the same matrix on every rank
            sets = [(torch.rand(M, device=device, generator=g) - 0.5, torch.rand(M, N, device=device, generator=g) - 0.5)
                    for _ in range(3)]
            slices = [(a, b[:, lo:hi].contiguous()) for a, b in sets]
            out = torch.empty(M, device=device)
            nbytes = lambda t: t.numel() * t.element_size()
            tiling = spec.pack({"M": M, "N": hi - lo})
            raw = stream.cuda_stream

            def local_only(i):
                a, mine = slices[i % 3]
                rt.launch_device(spec.binary, spec.name, [(a.data_ptr(), nbytes(a)), (mine.data_ptr(), nbytes(mine))],
                                 [(out.data_ptr(), nbytes(out))], tiling, 0, spec.magic, stream=raw)

            def two_step(i):
                local_only(i)
                dist.all_reduce(out)

            def fused(i):
                a, b = sets[i % 3]
                exchange.bcast_add_rowsum(a.data_ptr(), b.data_ptr() + lo * 4, out.data_ptr(), M, hi - lo, N, "f32", raw)

            two_step(0)
            want = out.clone()
            fused(0)
            stream.synchronize()
            try:
                exchange.check()
                close = bool(torch.allclose(out, want, rtol=1e-5, atol=1e-3))
                error = None if close else "the fused result differs from kernel + all-reduce"
            except Exception as e:
                error = f"{type(e).__name__}: {e}"
            if not all_ok(error is None):
                return {"error": error or "another rank failed the first exchange"}
            micros = {}
            for name, fn in (("slice_kernel_only", local_only), ("kernel_plus_nccl_allreduce", two_step), ("fused_exchange", fused)):
                for i in range(warmup):
                    fn(i)
                stream.synchronize()
                if name == "fused_exchange":
                    try:
                        exchange.check()
                    except Exception as e:
                        error = f"{type(e).__name__}: {e}"
                    if not all_ok(error is None):
                        return {"error": error or "another rank's exchange timed out"}
                dist.barrier()
                torch.cuda.synchronize(device)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for i in range(steps):
                    fn(i)
                e1.record(stream)
                stream.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                micros[name] = float(t.item()) * 1000.0
            exchange.check()
        work = M * N * 4 + 2 * M * 4  # the matrix once, the broadcast operand and the result
        return {"value": work / (micros["fused_exchange"] * 1e-6) / 1e9, "unit": "GB/s", "scaling": "strong",
                "shape": {"M": M, "N": N, "dtype": "f32"}, "steps": steps, "launches_per_step": 1.0,
                "microseconds_per_call": micros, "algorithmic_work_per_step": work,
                "exchange": "partial row sums stored into every rank's peer-mapped mailbox by the reduction kernel itself; "
                            "no library collective in the fused arm",
                "fused_speedup_over_nccl": micros["kernel_plus_nccl_allreduce"] / micros["fused_exchange"]}
    except Exception as e:
        return {"error": f"{type(e).__name__}: {e}"}
    finally:
        try:
            torch.cuda.synchronize(device)
            dist.barrier()
        finally:
            exchange.close()


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from ascend_mlir_b200.runtime.executor import CudaRuntime

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused-group kernels have no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()
    rt = CudaRuntime()
    rt.set_device(local)
    stream = torch.cuda.Stream(device)

    def sync():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    everything = {**configs.CONFIGS, **configs.EXTRA_CONFIGS}
    names = [args.workload] + ([n for n in everything if n != args.workload] if args.all_groups else [])
    results, main = {}, None
    sampler = ClockSampler(local)
    sampler.start()
    for name in names:
        try:
            # weak scaling: every rank owns one full-size batch (a distinct seed per rank)
            w = everything[name](seed=rank)
            g = DeviceGroup(torch, rt, w, device, stream, args.buffer_sets)
            steps = args.steps if name == args.workload else max(20, min(args.steps, 200))
            ms, launches = g.timed(steps, args.warmup, sync, use_graph=not args.no_graph)
            ms = max_over_ranks(ms)
            work, unit, scale = work_of(w)
            value = world * work / (ms * 1e-3) / scale
            rec = {"value": value, "unit": unit, "ms_per_step": ms, "launches_per_step": launches / steps,
                   "launch_mode": g.launch_mode,
                   "algorithmic_work_per_step": work}
            if name == args.workload:
                e2e_steps = max(3, min(steps, 20))
                ems = max_over_ranks(g.timed_e2e(e2e_steps, 2, sync))
                rec["e2e"] = {"value": world * work / (ems * 1e-3) / scale, "unit": unit, "ms_per_step": ems,
                              "h2d_bytes_per_step": int(sum(n for _, n in g.host_in_args)),
                              "d2h_bytes_per_step": int(sum(n for _, n in g.host_out_args))}
                rec["gpu_launches"] = int(launches)
                rec["steps"] = steps
                main = (w, rec)
            peak = (peaks["bf16_tflops_sustained"] if unit == "TFLOP/s" else peaks["hbm_gbs"])
            per_gpu = value / world
            rec["roofline"] = {"bound": "tensor" if unit == "TFLOP/s" else "hbm", "achieved": per_gpu, "peak": peak,
                               "unit": unit, "frac": per_gpu / peak, "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(name),
                               "peak_source": peaks["source"],
                               "frac_of_nominal": per_gpu / (NOMINAL_BF16_TFLOPS if unit == "TFLOP/s" else NOMINAL_HBM_GBS)}
            results[name] = rec
            del g
            torch.cuda.empty_cache()
        except Exception as e:  # a group that cannot run is reported, not hidden
            results[name] = {"error": f"{type(e).__name__}: {e}"}
            if name == args.workload:
                sampler.finish()
                raise
    if world > 1 and args.all_groups:
        results["broadcast_add_reduce_column_sharded"] = column_sharded_reduce(torch, dist, rt, device, stream, rank, world, local)
    clocks = sampler.finish()

    if rank == 0:
        w, rec = main
        line = {"metric": METRIC, "value": rec["value"], "unit": rec["unit"], "n_gpus": world, "steps": rec["steps"],
                "warmup": args.warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": dtype_of(args.workload), "data": "synthetic",
                "config": {"workload": args.workload, "shape": w.shape, "per_gpu_batches": 1,
                           "sharding": "leading axis row-sharded, one full-size batch per GPU, no collective",
                           "l2": f"{args.buffer_sets} device buffer sets used in rotation (a step touches memory last used "
                                 f"{args.buffer_sets} steps earlier); the per-step working set also exceeds the 126 MB L2",
                           "launch_mode": rec["launch_mode"],
                           "notes": w.notes},
                "roofline": rec["roofline"], "e2e": rec["e2e"], "gpu_launches": rec["gpu_launches"], "clocks": clocks,
                "groups": {k: v for k, v in results.items() if k != args.workload}}
        if world == 1 and not args.no_cpu:
            cpu, _ = time_cpu(args.workload, 3, 1)
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=list(configs.CONFIGS) + list(configs.EXTRA_CONFIGS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--one-group", dest="all_groups", action="store_false", help="time only --workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the host-CPU baseline leg")
    ap.add_argument("--buffer-sets", type=int, default=3, help="identical device buffer sets per group, used in rotation")
    ap.add_argument("--no-graph", action="store_true", help="issue the timed launches one by one instead of replaying a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
