#!/usr/bin/env python3
"""Benchmark of the fused-group hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of one fused group over one batch of seeded synthetic input.  The default workload is the
split-relu-broadcast-add-mul group (f16 [32,1024,2048] -> [32,1024,1024]); the other four benchmark groups, three
transpose-class groups and three generic chains (bodies that run on the kernel GENERATED for the group) are timed
the same way and reported under "groups".

  value     device-resident throughput: the K launches of a step sequence are captured into a CUDA graph, the graph
            is replayed several times and the median replay is the figure (CUDA events on the launching stream)
  e2e       the same pass through afirt_executor_run with pinned HOST buffers (H2D + kernel + D2H in the timed
            region); e2e_pageable the same with ordinary (pageable) host arrays, which is what a numpy caller has
  roofline  algorithmic bytes (or flops) / device time against the measured peaks of MEASURED_PEAKS.json
  cpu_baseline  the CPU restatement of the reference semantics on the host cores (every group at N = 1)

With N > 1 (torchrun, one rank per GPU) the headline is weak scaling -- every rank runs a full-size batch of its
own, the leading axis grows with N and is sharded row-wise, no collective -- and every group also carries a
"strong" record: the ONE full-size configuration cut into N contiguous row shards (matmul: A and the output
M-sharded, B and bias replicated; gather: table replicated), value = the fixed total work / the slowest rank.
`--impl reference` times the CPU restatement of the reference semantics on the host cores instead.
"""
import argparse
import json
import os
import re
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
REPLAYS = 7                 # graph replays per timed group; the median one is reported
BURST_REGION_SECONDS = 0.1  # a tensor-bound region shorter than this runs at boost clocks: compare with the burst peak
CPU_BUDGET_SECONDS = 20.0   # per group, host-CPU leg


def dram_traffic_table():
    """workload -> DRAM bytes per launch, from the committed table of ncu captures (never measured here)."""
    table = {}
    path = ROOT / "profiles" / "dram_traffic_per_launch.md"
    if path.exists():
        for line in path.read_text().splitlines():
            m = re.match(r"^\|\s*([a-z0-9_]+)\s*\|[^|]*\|\s*(\d+)\s*\|\s*(\d+)\s*\|", line)
            if m:
                table[m.group(1)] = int(m.group(2))
    return table


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


def bind_to_gpu_numa_node(index: int):
    """Pins this process to the CPUs NVML lists as local to GPU `index` (a read-only query), before any pinned host
    buffer is allocated, so that on a box with several NUMA nodes a rank's host buffers sit next to its GPU.
    Returns a short description for the output line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (int(w) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        cpus &= allowed
        if cpus and cpus != allowed:
            os.sched_setaffinity(0, cpus)
            return {"bound": True, "cpus": len(cpus)}
        return {"bound": False, "cpus": len(allowed), "note": "every allowed CPU is local to this GPU (one NUMA node)"}
    except Exception as e:
        return {"bound": False, "note": f"affinity not available: {type(e).__name__}"}


# ---- workloads and the CPU restatement ---------------------------------------------------------------------------------
def all_workloads():
    return {**configs.CONFIGS, **configs.EXTRA_CONFIGS, **configs.GENERIC_CHAINS}


def dtype_of(name):
    return {"elementwise_chain": "f32", "split_relu_broadcast_add_mul": "f16", "broadcast_add_reduce": "f32",
            "gather_elementwise": "bf16", "matmul_add_leakyrelu": "bf16", "transpose_2d": "f16",
            "relu_broadcast_transpose_add": "f16", "transposed_add_mul": "f16"}.get(name, "f32")


def cpu_sample(name: str):
    """A bounded sample of the workload for the host-CPU leg: (workload, callable, description, extrapolation note)."""
    from oracle import oracle
    if name == "elementwise_chain":
        w = configs.elementwise_chain()
        return w, (lambda: oracle.add_mul_f32(*w.inputs)), "full config, f32 [4096,4096]", None
    if name == "split_relu_broadcast_add_mul":
        w = configs.split_relu_broadcast_add_mul()
        return w, (lambda: oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], 1)), "full config, f16 [32,1024,2048]", None
    if name == "broadcast_add_reduce":
        w = configs.broadcast_add_reduce()
        return w, (lambda: oracle.bcast_add_rowsum_f32(w.inputs[0], w.inputs[1])), "full config, f32 [8192,8192]", None
    if name == "gather_elementwise":
        w = configs.gather_elementwise()
        return w, (lambda: oracle.gather_rows_scale_resid_bf16(*w.inputs)), "full config, 262144 rows of a 1M-row table", None
    if name == "matmul_add_leakyrelu":
        w = configs.matmul_add_leakyrelu(M=256)
        return (w, (lambda: oracle.matmul_bias_leakyrelu_bf16(*w.inputs, 0.01)), "256 of 8192 output rows (N=K=8192)",
                "extrapolated from 256 rows: the rate is per row of A, the full 8192-row problem takes 32 x as long")
    if name == "transpose_2d":
        w = configs.transpose_2d()
        return w, (lambda: oracle.transpose_2d(w.inputs[0])), "full size, f16 [8192,8192]", None
    if name == "relu_broadcast_transpose_add":
        w = configs.relu_broadcast_transpose_add()
        return w, (lambda: oracle.relu_bcast_transpose_add_f16(*w.inputs)), "full size, f16 [8192,8192]", None
    if name == "transposed_add_mul":
        w = configs.transposed_add_mul()
        return w, w.expected, "full size, f16 [8192,8192] (numpy, one pass per op)", None
    if name in configs.GENERIC_CHAINS and name != "chain_torch_model":
        w = configs.GENERIC_CHAINS[name]()
        return w, w.expected, "full size, f32 [4096,4096] (numpy, one pass per op, all cores of its BLAS-free ufuncs)", None
    return None


def work_of(w):
    return (w.flops, "TFLOP/s", 1e12) if w.bound == "tensor" else (w.algorithmic_bytes, "GB/s", 1e9)


def time_cpu(name: str, steps: int, warmup: int, budget_s: float = CPU_BUDGET_SECONDS):
    """The CPU restatement on every host core: `warmup` untimed passes, then up to `steps` timed ones inside the time budget."""
    # torchrun exports OMP_NUM_THREADS=1; the CPU leg is meant to use every host core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from oracle import oracle
    oracle.set_num_threads(os.cpu_count() or 1)
    sample = cpu_sample(name)
    if sample is None:
        return None, None
    w, fn, what, extrapolated = sample
    deadline = time.time() + budget_s
    for _ in range(max(1, warmup)):
        fn()
        if time.time() > deadline:
            break
    times = []
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
        if time.time() > deadline:
            break
    work, unit, scale = work_of(w)
    best = min(times)
    rec = {"value": work / best / scale, "unit": unit, "cores": oracle.num_threads(), "kind": "port", "sample": what,
           "seconds_per_pass": best, "passes": len(times)}
    if w.expected is not None:
        rec["cores"] = 1  # plain numpy ufuncs: one thread
    if extrapolated:
        rec["extrapolated"] = extrapolated
    return rec, w


def shared_config(name: str, w, buffer_sets: int):
    """The `config` object of the JSON line: identical in the GPU arm and the reference arm."""
    ws_mib = (sum(int(x.nbytes) for x in w.inputs) + int(np.prod(w.out_shape)) * np.dtype(w.out_dtype).itemsize) / 2 ** 20
    return {"workload": name, "shape": w.shape, "notes": w.notes,
            "l2": f"inputs larger than L2: the per-step working set is {ws_mib:.0f} MiB against 126 MB of L2; the GPU arm "
                  f"also rotates {buffer_sets} identical device buffer sets, so a step touches memory last used {buffer_sets} steps earlier"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu, w = time_cpu(args.workload, args.steps, args.warmup, budget_s=150.0)
    if cpu is None:
        print(json.dumps({"impl": "reference", "unavailable": f"no CPU restatement of workload {args.workload}"}), flush=True)
        return
    full = all_workloads()[args.workload]() if args.workload == "matmul_add_leakyrelu" else w
    line = {"metric": METRIC, "value": cpu["value"], "unit": cpu["unit"], "n_gpus": args.gpus, "steps": cpu["passes"],
            "warmup": args.warmup, "ms_per_step": cpu["seconds_per_pass"] * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype_of(args.workload), "data": "synthetic", "impl": "reference",
            "config": shared_config(args.workload, full, args.buffer_sets),
            "measurement": {"what": "CPU restatement of the reference semantics (the reference's own device path needs MLIR + CANN "
                                    "and cannot be built here), OpenMP over all host cores; best pass of `steps`",
                            "steps_requested": args.steps, "time_budget_s": 150.0},
            "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample") if k in cpu},
            "e2e": {"value": cpu["value"], "unit": cpu["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if "extrapolated" in cpu:
        line["cpu_baseline"]["extrapolated"] = cpu["extrapolated"]
    print(json.dumps(line), flush=True)


# ---- GPU arm ------------------------------------------------------------------------------------------------
def as_torch(torch, x):
    x = np.ascontiguousarray(x)
    if x.dtype in (np.uint16, np.float16):
        x = x.view(np.int16)
    return torch.from_numpy(x)


class DeviceGroup:
    """One workload resident on the device, launched through the C-ABI device entry point."""

    def __init__(self, torch, rt, w, device, stream, buffer_sets=3, pinned=True):
        self.torch, self.rt, self.w, self.stream = torch, rt, w, stream
        self.host_in = [as_torch(torch, x) for x in w.inputs]
        if pinned:
            self.host_in = [t.pin_memory() for t in self.host_in]
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
        self.host_out = torch.empty(tuple(w.out_shape), dtype=self.dev_out.dtype)
        if pinned:
            self.host_out = self.host_out.pin_memory()
        self.turn = 0
        self.tiling = w.tiling()
        ws_bytes = rt.workspace_bytes(w.spec.binary, self.tiling)
        self.ws = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=device)
        self.host_in_args = [(t.data_ptr(), t.numel() * t.element_size()) for t in self.host_in]
        self.host_out_args = [(self.host_out.data_ptr(), self.host_out.numel() * self.host_out.element_size())]
        self.generated = None

    def launch(self, cuda_stream=None):
        _, _, in_args, out_args = self.sets[self.turn % len(self.sets)]
        self.turn += 1
        self.rt.launch_device(self.w.spec.binary, self.w.spec.name, in_args, out_args, self.tiling, 0, self.w.spec.magic,
                              (self.ws.data_ptr(), self.ws.numel()),
                              self.stream.cuda_stream if cuda_stream is None else cuda_stream)

    def last_output(self):
        return self.sets[(self.turn - 1) % len(self.sets)][1]

    def run_host(self, host_in_args=None, host_out_args=None):
        self.rt.run_raw(self.w.spec.binary, self.w.spec.name, host_in_args or self.host_in_args, host_out_args or self.host_out_args,
                        self.tiling, 0, self.w.spec.magic)

    def timed(self, steps, warmup, sync, use_graph=True, replays=REPLAYS):
        """Milliseconds per step (median over `replays` timed replays of a CUDA graph holding the K launches), the
        launches per replay, and the spread.  If capture is refused the launches are issued one by one through the
        C-ABI, `replays` times, and the median sequence is reported the same way."""
        torch = self.torch
        for _ in range(warmup):
            self.launch()
        sync()
        self.generated = bool(self.rt.last_launch_generated)
        graph, mode = None, "direct"
        launches = steps
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
        times = []
        for _ in range(max(1, replays)):
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
            times.append(e0.elapsed_time(e1) / steps)
        self.rt.synchronize(self.stream.cuda_stream)
        self.launch_mode = mode
        times.sort()
        self.spread = {"replays": len(times), "min_ms": times[0], "max_ms": times[-1]}
        return times[len(times) // 2], launches

    def timed_burst(self, sync, launches=20, pause_s=3.0, repeats=3):
        """Tensor-bound groups: milliseconds per launch of ONE short graph replay started after a pause, i.e. at boost
        clocks before the board's power cap bites (it does within about 60 launches of the 8192^3 GEMM).  Median of
        `repeats` such replays.  The long timed region of timed() reports the power-capped regime; this is the other one."""
        torch = self.torch
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=self.stream, capture_error_mode="thread_local"):
            for _ in range(launches):
                self.launch(torch.cuda.current_stream().cuda_stream)
        with torch.cuda.stream(self.stream):
            g.replay()
        sync()
        times = []
        for _ in range(repeats):
            time.sleep(pause_s)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(self.stream):
                e0.record(self.stream)
                g.replay()
                e1.record(self.stream)
            sync()
            times.append(e0.elapsed_time(e1) / launches)
        times.sort()
        return times[len(times) // 2], launches

    def timed_e2e(self, steps, warmup, sync, host_in_args=None, host_out_args=None):
        for _ in range(warmup):
            self.run_host(host_in_args, host_out_args)
        sync()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.run_host(host_in_args, host_out_args)
        sync()
        return (time.perf_counter() - t0) * 1e3 / steps


def host_copy_ceiling(torch, device, sync, world, nbytes=256 << 20, repeats=4):
    """What the box gives pinned host<->device copies when every rank copies at once: H2D alone, D2H alone and both
    directions together (GB/s per rank, slowest rank).  The end-to-end leg cannot beat these."""
    host_a = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    host_b = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dev_a = torch.empty(nbytes, dtype=torch.uint8, device=device)
    dev_b = torch.empty(nbytes, dtype=torch.uint8, device=device)
    s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def run(h2d, d2h):
        sync()
        t0 = time.perf_counter()
        for _ in range(repeats):
            if h2d:
                with torch.cuda.stream(s1):
                    dev_a.copy_(host_a, non_blocking=True)
            if d2h:
                with torch.cuda.stream(s2):
                    host_b.copy_(dev_b, non_blocking=True)
        s1.synchronize()
        s2.synchronize()
        dt = time.perf_counter() - t0
        return repeats * nbytes / dt / 1e9

    run(True, True)
    out = {"h2d_gbs": run(True, False), "d2h_gbs": run(False, True)}
    both = run(True, True)
    out["both_directions_gbs_each"] = both
    out["ranks_copying_at_once"] = world
    return out


def column_sharded_reduce(torch, dist, rt, device, stream, rank, world, local, steps=200, warmup=10):
    """The one exchange step the path has: broadcast_add_reduce with its REDUCED axis sharded (strong scaling,
    one 8192 x 8192 f32 matrix, every rank reads its column slice in place).  Times the slice kernel alone, the
    slice kernel followed by an NCCL all-reduce of the partial sums, and the kernel that exchanges the partial
    sums itself through peer-mapped mailboxes; the fused result is also checked against the f64 row sums within the
    oracle's bound 1e-5 * sum|x| (`max_abs_err_over_bound` <= 1).  Every step that can fail on one rank only is
    followed by a MIN over ranks, so either all ranks go on or all stop; the waits inside the kernel are bounded."""
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
            over_bound = None
            try:
                exchange.check()
                close = bool(torch.allclose(out, want, rtol=1e-5, atol=1e-3))
                error = None if close else "the fused result differs from kernel + all-reduce"
                # parity against exact arithmetic: out[m] = sum_n (a[m] + b[m, n]) over the WHOLE row
                a0, b0 = sets[0]
                terms = a0.double()[:, None] + b0.double()
                exact, bound = terms.sum(dim=1), 1e-5 * terms.abs().sum(dim=1)
                over_bound = float(((out.double() - exact).abs() / bound).max().item())
                if over_bound > 1.0:
                    error = f"the fused result is {over_bound:.2f} x outside the 1e-5 * sum|x| bound"
            except Exception as e:
                error = f"{type(e).__name__}: {e}"
            if not all_ok(error is None):
                return {"error": error or "another rank failed the first exchange"}
            # How each arm's `steps` calls are issued, so that the figure is device time and not the cost of calling
            # through Python: the slice kernel alone and the fused exchange (whose call number lives on the device, so
            # a replay continues the sequence) are each captured into a CUDA graph and replayed; kernel + NCCL stays a
            # Python loop (its all-reduce dominates anyway).  If a capture is refused on any rank, every rank falls
            # back to one call of the batch entry point.
            def fused_batch(n):
                picks = [sets[i % 3] for i in range(n)]
                exchange.bcast_add_rowsum_batch([a.data_ptr() for a, _ in picks], [b.data_ptr() + lo * 4 for _, b in picks],
                                                [out.data_ptr()] * n, M, hi - lo, N, "f32", raw)

            slice_graph = None
            try:
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=stream, capture_error_mode="thread_local"):
                    cap = torch.cuda.current_stream().cuda_stream
                    for i in range(steps):
                        a, mine = slices[i % 3]
                        rt.launch_device(spec.binary, spec.name, [(a.data_ptr(), nbytes(a)), (mine.data_ptr(), nbytes(mine))],
                                         [(out.data_ptr(), nbytes(out))], tiling, 0, spec.magic, stream=cap)
                slice_graph = g_
            except Exception:
                slice_graph = None
            fused_graph = None
            try:
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=stream, capture_error_mode="thread_local"):
                    cap = torch.cuda.current_stream().cuda_stream
                    picks = [sets[i % 3] for i in range(steps)]
                    exchange.bcast_add_rowsum_batch([a.data_ptr() for a, _ in picks], [b.data_ptr() + lo * 4 for _, b in picks],
                                                    [out.data_ptr()] * steps, M, hi - lo, N, "f32", cap)
                fused_graph = g_
            except Exception:
                fused_graph = None
            if not all_ok(fused_graph is not None):  # every rank must issue the same number of calls the same way
                fused_graph = None
            issue = {"slice_kernel_only": "cuda_graph" if slice_graph is not None else "python loop",
                     "kernel_plus_nccl_allreduce": "python loop",
                     "fused_exchange": "cuda_graph" if fused_graph is not None else "one batch call"}
            micros = {}
            for name, fn in (("slice_kernel_only", local_only), ("kernel_plus_nccl_allreduce", two_step), ("fused_exchange", fused)):
                for i in range(warmup):
                    fn(i)
                graph_ = slice_graph if name == "slice_kernel_only" else fused_graph if name == "fused_exchange" else None
                if graph_ is not None:  # one untimed replay: the graph's upload stays out of the timing
                    with torch.cuda.stream(stream):
                        graph_.replay()
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
                if name == "slice_kernel_only" and slice_graph is not None:
                    slice_graph.replay()
                elif name == "fused_exchange" and fused_graph is not None:
                    fused_graph.replay()
                elif name == "fused_exchange":
                    fused_batch(steps)
                else:
                    for i in range(steps):
                        fn(i)
                e1.record(stream)
                stream.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                micros[name] = float(t.item()) * 1000.0
            exchange.check()
            worst = torch.tensor([over_bound], dtype=torch.float64, device=device)
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        work = M * N * 4 + 2 * M * 4  # the matrix once, the broadcast operand and the result
        slice_bytes = M * (hi - lo) * 4
        return {"value": work / (micros["fused_exchange"] * 1e-6) / 1e9, "unit": "GB/s", "scaling": "strong",
                "shape": {"M": M, "N": N, "dtype": "f32"}, "steps": steps, "launches_per_step": 1.0,
                "microseconds_per_call": micros, "issued_as": issue, "algorithmic_work_per_step": work,
                "slice_kernel_gbs_per_gpu": slice_bytes / (micros["slice_kernel_only"] * 1e-6) / 1e9,
                "max_abs_err_over_bound": float(worst.item()),
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


def exchange_world_of_one(torch, rt, device, stream, local, peaks, traffic, steps=200, warmup=5):
    """One GPU: the reduction kernel that exchanges its partial sums itself, with a world of one rank (its mailbox is
    its own memory), beside the ordinary reduction kernel on the same 8192 x 8192 f32 matrix.  The difference is what
    the exchange costs inside the kernel (ticket, sends, the wait for the entries) before any NVLink latency; the
    result is compared bit for bit with the ordinary kernel's.  Both arms are CUDA graphs of `steps` launches."""
    from ascend_mlir_b200 import descriptors, sharding
    M = N = 8192
    spec = descriptors.bcast_add_rowsum("f32")
    exchange = None
    try:
        exchange = sharding.RowsumExchange(local, 0, 1, max_rows=M)
        exchange.connect()
        nbytes = lambda t: t.numel() * t.element_size()
        with torch.cuda.stream(stream):
            sets = [(torch.rand(M, device=device) - 0.5, torch.rand(M, N, device=device) - 0.5) for _ in range(3)]
            out = [torch.empty(M, device=device), torch.empty(M, device=device)]
            tiling = spec.pack({"M": M, "N": N})

            def ordinary(s, n):
                for i in range(n):
                    a, b = sets[i % 3]
                    rt.launch_device(spec.binary, spec.name, [(a.data_ptr(), nbytes(a)), (b.data_ptr(), nbytes(b))],
                                     [(out[0].data_ptr(), nbytes(out[0]))], tiling, 0, spec.magic, stream=s)

            def fused(s, n):
                picks = [sets[i % 3] for i in range(n)]
                exchange.bcast_add_rowsum_batch([a.data_ptr() for a, _ in picks], [b.data_ptr() for _, b in picks],
                                                [out[1].data_ptr()] * n, M, N, N, "f32", s)

            micros = {}
            for name, fn in (("ordinary_kernel", ordinary), ("exchange_kernel", fused)):
                fn(stream.cuda_stream, max(warmup, 1))  # set-up and warm-up outside the capture
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                    fn(torch.cuda.current_stream().cuda_stream, steps)
                times = []
                for _ in range(REPLAYS + 1):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    graph.replay()
                    e1.record(stream)
                    stream.synchronize()
                    times.append(e0.elapsed_time(e1) / steps * 1000.0)
                times = sorted(times[1:])  # the first replay uploads the graph
                micros[name] = times[len(times) // 2]
            exchange.check()
            same = bool(torch.equal(out[0], out[1]))  # both hold the sums of buffer set (steps - 1) % 3
        work = M * N * 4 + 2 * M * 4
        gbs = work / (micros["exchange_kernel"] * 1e-6) / 1e9
        return {"value": gbs, "unit": "GB/s", "shape": {"M": M, "N": N, "dtype": "f32"}, "steps": steps, "launches_per_step": 1.0,
                "launch_mode": "cuda_graph", "microseconds_per_call": micros, "algorithmic_work_per_step": work,
                "bit_equal_to_ordinary_kernel": same, "code": "library",
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                             "traffic": traffic.get("broadcast_add_reduce_exchange_world_of_one"), "peak_source": peaks["source"],
                             "frac_of_nominal": gbs / NOMINAL_HBM_GBS},
                "note": "world of one rank: the exchange's cost inside the kernel, no NVLink; the multi-GPU figures are in "
                        "groups.broadcast_add_reduce_column_sharded of a --gpus N run"}
    except Exception as e:
        return {"error": f"{type(e).__name__}: {e}"}
    finally:
        if exchange is not None:
            try:
                torch.cuda.synchronize(device)
            finally:
                exchange.close()


def roofline_of(name, unit, per_gpu, region_seconds, peaks, traffic):
    if unit == "TFLOP/s":
        # a short region runs at boost clocks, a long one settles under the board's power cap: compare like with like
        burst = region_seconds < BURST_REGION_SECONDS
        peak = peaks["bf16_tflops"] if burst else peaks["bf16_tflops_sustained"]
        return {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": unit, "frac": per_gpu / peak,
                "peak_kind": "burst" if burst else "sustained", "timed_region_s": region_seconds,
                "frac_of_burst": per_gpu / peaks["bf16_tflops"], "frac_of_sustained": per_gpu / peaks["bf16_tflops_sustained"],
                "traffic": traffic.get(name), "peak_source": peaks["source"], "frac_of_nominal": per_gpu / NOMINAL_BF16_TFLOPS}
    return {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": unit, "frac": per_gpu / peaks["hbm_gbs"],
            "traffic": traffic.get(name), "peak_source": peaks["source"], "frac_of_nominal": per_gpu / NOMINAL_HBM_GBS}


def run_gpu_arm(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    affinity = bind_to_gpu_numa_node(local)  # before torch allocates any pinned memory

    import torch
    import torch.distributed as dist
    from ascend_mlir_b200.runtime.executor import CudaRuntime

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused-group kernels have no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()
    traffic = dram_traffic_table()
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

    def all_ranks(flag):
        if world == 1:
            return flag
        t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    everything = all_workloads()
    names = [args.workload] + ([n for n in everything if n != args.workload] if args.all_groups else [])
    if args.exchange_only:
        names = []
    results, main = {}, None
    weak_workloads = {}
    sampler = ClockSampler(local)
    sampler.start()
    for name in names:
        try:
            # weak scaling: every rank owns one full-size batch (a distinct seed per rank)
            w = everything[name](seed=rank)
            # host buffers are pinned only where the end-to-end leg needs them (pinning 0.5 GB per group costs seconds)
            g = DeviceGroup(torch, rt, w, device, stream, args.buffer_sets, pinned=name == args.workload)
            steps = args.steps if name == args.workload else max(20, min(args.steps, 200))
            ms, launches = g.timed(steps, args.warmup, sync, use_graph=not args.no_graph)
            ms = max_over_ranks(ms)
            weak_workloads[name] = w
            work, unit, scale = work_of(w)
            value = world * work / (ms * 1e-3) / scale
            rec = {"value": value, "unit": unit, "ms_per_step": ms, "launches_per_step": launches / steps,
                   "launch_mode": g.launch_mode, "timing": g.spread, "algorithmic_work_per_step": work,
                   "code": "generated" if g.generated else "library"}
            if w.expected is not None:  # generic chains: the bench checks its own result, bit for bit
                got = g.last_output().cpu().numpy()
                rec["bit_exact_vs_numpy"] = bool(np.array_equal(got.view(np.uint32), np.ascontiguousarray(w.expected()).view(np.uint32)))
            if name == args.workload:
                e2e_steps = max(3, min(steps, 20))
                ems = max_over_ranks(g.timed_e2e(e2e_steps, 2, sync))
                h2d = int(sum(n for _, n in g.host_in_args))
                d2h = int(sum(n for _, n in g.host_out_args))
                rec["e2e"] = {"value": world * work / (ems * 1e-3) / scale, "unit": unit, "ms_per_step": ems,
                              "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                              "h2d_gbs_per_gpu": h2d / (ems * 1e-3) / 1e9, "d2h_gbs_per_gpu": d2h / (ems * 1e-3) / 1e9,
                              "host_buffers": "pinned"}
                # the same call with ordinary pageable host arrays (what a numpy caller hands to afirt_executor_run)
                pageable_in = [as_torch(torch, x).clone() for x in w.inputs]
                pageable_out = torch.empty(tuple(w.out_shape), dtype=g.dev_out.dtype)
                pin = [(t.data_ptr(), t.numel() * t.element_size()) for t in pageable_in]
                pout = [(pageable_out.data_ptr(), pageable_out.numel() * pageable_out.element_size())]
                pms = max_over_ranks(g.timed_e2e(max(3, min(steps, 8)), 1, sync, pin, pout))
                rec["e2e_pageable"] = {"value": world * work / (pms * 1e-3) / scale, "unit": unit, "ms_per_step": pms,
                                       "host_buffers": "pageable"}
                rec["e2e"]["host_copy_ceiling"] = host_copy_ceiling(torch, device, sync, world)
                rec["gpu_launches"] = int(launches)
                rec["steps"] = steps
                main = (w, rec)
            rec["roofline"] = roofline_of(name, unit, value / world, REPLAYS * steps * ms * 1e-3, peaks, traffic)
            if unit == "TFLOP/s":
                # the same kernel in the other regime: one short replay after a pause, against the library's burst figure
                bms, blaunches, berr = 0.0, 0, None
                try:
                    bms, blaunches = g.timed_burst(sync)
                except Exception as e:
                    berr = f"{type(e).__name__}: {e}"
                try:
                    if not all_ranks(berr is None):  # every rank goes on, or none
                        raise RuntimeError(berr or "another rank failed")
                    bms = max_over_ranks(bms)
                    per_gpu = work / (bms * 1e-3) / scale
                    rec["burst"] = {"value": world * per_gpu, "unit": unit, "ms_per_step": bms, "launches": blaunches, "pause_s": 3.0,
                                    "frac_of_burst_peak": per_gpu / peaks["bf16_tflops"], "frac_of_nominal": per_gpu / NOMINAL_BF16_TFLOPS,
                                    "note": "one graph replay of `launches` launches after a pause (boost clocks); `value` above is the "
                                            "median of back-to-back replays (power-capped)"}
                except Exception as e:
                    rec["burst"] = {"error": f"{type(e).__name__}: {e}"}
            if name in traffic and traffic[name] < work and unit == "GB/s":
                rec["roofline"]["traffic_note"] = "single launch under ncu: part of the output was still dirty in L2 when the counters stopped"
            results[name] = rec
            del g
            torch.cuda.empty_cache()
        except Exception as e:  # a group that cannot run is reported, not hidden
            results[name] = {"error": f"{type(e).__name__}: {e}"}
            if name == args.workload:
                sampler.finish()
                raise

    # Strong scaling of the stated configurations: ONE full-size problem cut into contiguous row shards.
    if world > 1 and args.all_groups:
        floor_us = None
        for name in configs.CONFIGS:
            rec = results.get(name)
            if not isinstance(rec, dict) or "error" in rec:
                continue
            error = None
            ms = 0.0
            try:
                # shard `rank` of a full-size problem: every rank cuts it out of the full-size tensors it already holds
                # (its own seed: same shapes and value distributions as any other draw; generating them again costs
                # more than every timed region of this run together)
                full = weak_workloads[name]
                mine = full.shard(rank, world)
                # a shard is small: rotate enough buffer sets that a step's memory was last used >= 2 x L2 of traffic ago
                # (what a step streams: the algorithmic bytes; a replicated gather table is read at random and does not count)
                touched = mine.algorithmic_bytes if mine.bound == "hbm" and mine.algorithmic_bytes else (
                    sum(x.nbytes for x in mine.inputs) + int(np.prod(mine.out_shape)) * mine.out_dtype.itemsize)
                n_sets = int(min(12, max(args.buffer_sets, -(-2 * 126_000_000 // max(touched, 1)))))
                g = DeviceGroup(torch, rt, mine, device, stream, n_sets, pinned=False)
                steps = max(20, min(args.steps, 200))
                ms, _ = g.timed(steps, args.warmup, sync, use_graph=not args.no_graph)
                del g
                torch.cuda.empty_cache()
                if floor_us is None:  # what one more launch in a replayed graph costs when it moves almost nothing
                    tiny = DeviceGroup(torch, rt, configs.elementwise_chain(8, 1024), device, stream, 1, pinned=False)
                    floor_ms, _ = tiny.timed(200, args.warmup, sync, use_graph=not args.no_graph)
                    floor_us = floor_ms * 1e3
                    del tiny
            except Exception as e:
                error = f"{type(e).__name__}: {e}"
            if not all_ranks(error is None):
                rec["strong"] = {"error": error or "another rank failed"}
                continue
            ms = max_over_ranks(ms)
            work, unit, scale = work_of(full)
            value = work / (ms * 1e-3) / scale
            single = rec["value"] / world  # this run's per-GPU figure on a full-size batch
            rec["strong"] = {"value": value, "unit": unit, "ms_per_step": ms, "scaling": "strong",
                             "rows_per_gpu": mine.units, "total_work_per_step": work, "buffer_sets": n_sets,
                             "launch_floor_us": floor_us,
                             "per_gpu": value / world, "per_gpu_frac_of_full_batch_rate": (value / world) / single,
                             "sharding": "contiguous row shards of one full-size configuration, no collective (rank r times "
                                         "shard r; table, B and bias replicated)"}
        results["broadcast_add_reduce_column_sharded"] = column_sharded_reduce(torch, dist, rt, device, stream, rank, world, local)
    if world == 1 and (args.all_groups or args.exchange_only):
        results["broadcast_add_reduce_exchange_world_of_one"] = exchange_world_of_one(
            torch, rt, device, stream, local, peaks, traffic, steps=max(3, min(args.steps, 200)), warmup=min(args.warmup, 5))
    clocks = sampler.finish()
    if args.exchange_only:
        print(json.dumps({"groups": {"broadcast_add_reduce_exchange_world_of_one": results["broadcast_add_reduce_exchange_world_of_one"]},
                          "clocks": clocks}), flush=True)
        return

    if rank == 0:
        w, rec = main
        line = {"metric": METRIC, "value": rec["value"], "unit": rec["unit"], "n_gpus": world, "steps": rec["steps"],
                "warmup": args.warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": dtype_of(args.workload), "data": "synthetic",
                "config": shared_config(args.workload, w, args.buffer_sets),
                "measurement": {"per_gpu_batches": 1, "launch_mode": rec["launch_mode"], "timing": rec["timing"], "code": rec["code"],
                                "sharding": "leading axis row-sharded, one full-size batch per GPU, no collective",
                                "host_affinity": affinity},
                "roofline": rec["roofline"], "e2e": rec["e2e"], "e2e_pageable": rec["e2e_pageable"],
                **({"strong": rec["strong"]} if "strong" in rec else {}),
                **({"burst": rec["burst"]} if "burst" in rec else {}),
                "gpu_launches": rec["gpu_launches"], "clocks": clocks,
                "groups": {k: v for k, v in results.items() if k != args.workload}}
        if world == 1 and not args.no_cpu:
            cpu, _ = time_cpu(args.workload, 3, 1)
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
            for name, grec in line["groups"].items():  # beside every group, bounded
                if not isinstance(grec, dict) or "error" in grec:
                    continue
                gcpu, _ = time_cpu(name, 2, 1)
                if gcpu is not None:
                    grec["cpu_baseline"] = {k: gcpu[k] for k in ("value", "unit", "cores", "kind", "sample", "extrapolated") if k in gcpu}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=list(all_workloads()))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--one-group", dest="all_groups", action="store_false", help="time only --workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the host-CPU baseline legs")
    ap.add_argument("--exchange-only", action="store_true",
                    help="N=1: time only the world-of-one exchange kernel beside the ordinary reduction kernel")
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
