"""The host side of bench.py, without a GPU: the table of timed groups is complete (element type, CPU sample, DRAM
traffic row, sharder), and the reference arm prints the JSON line the driver parses."""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from ascend_mlir_b200 import configs

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("afir_bench", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_every_timed_group_has_an_element_type_and_a_cpu_sample(bench):
    names = list(bench.all_workloads())
    assert names[:5] == list(configs.CONFIGS) and "transposed_add_mul" in names and "transpose_2d" in names
    for name in names:
        assert bench.dtype_of(name) in ("f32", "f16", "bf16")
    # the CPU sample: every group but the traced torch module (its expected output comes from eager torch at trace time)
    for name in names:
        if name == "chain_torch_model":
            continue
        sample = bench.cpu_sample(name)
        assert sample is not None, f"{name}: no CPU sample in bench.cpu_sample"
        w, fn, what, _ = sample
        assert w.name == name and callable(fn) and what


def test_the_traffic_table_has_a_row_for_every_timed_group(bench):
    table = bench.dram_traffic_table()
    for name in bench.all_workloads():
        assert name in table and table[name] > 0, name
    assert "broadcast_add_reduce_exchange_world_of_one" in table


@pytest.mark.parametrize("name,small", [("transpose_2d", dict(R=24, C=40)), ("relu_broadcast_transpose_add", dict(M=16, N=24)),
                                        ("transposed_add_mul", dict(M=16, N=24)), ("chain_sub_div_min", dict(M=24, N=16)),
                                        ("chain_six_ops", dict(M=24, N=16))])
def test_small_instances_of_the_extra_groups_are_consistent(bench, name, small):
    w = bench.all_workloads()[name](**small)
    work, unit, scale = bench.work_of(w)
    assert unit == "GB/s" and scale == 1e9
    moved = sum(int(x.nbytes) for x in w.inputs) + int(np.prod(w.out_shape)) * np.dtype(w.out_dtype).itemsize
    assert work == moved  # every operand is read once and the output written once
    if w.sharder is not None:
        parts = [w.shard(r, 3) for r in range(3)]
        assert sum(p.units for p in parts) == w.units
        assert sum(bench.work_of(p)[0] for p in parts) >= work  # (a replicated operand counts once per shard)
        for p in parts:
            assert p.spec is w.spec and tuple(p.out_shape)[0] == p.units


def test_reference_arm_prints_the_line_the_driver_parses():
    """`bench.py --impl reference`: the CPU restatement on the host cores, same metric / unit / config keys as the GPU
    arm, `impl`, a `cpu_baseline` describing this very run and an `e2e` that repeats the line's value with no copies."""
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == bench_metric() and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["vs_baseline"] is None
    assert line["config"]["workload"] == "split_relu_broadcast_add_mul" and line["dtype"] == "f16"
    cpu = line["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == line["value"] and cpu["sample"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
    assert line["value"] > 0 and line["ms_per_step"] > 0


def bench_metric():
    return "fused_group_hbm_throughput"


def test_reference_arm_under_torchrun_prints_once_and_every_rank_exits_zero():
    """Launched like the GPU arm for N = 2: rank 0 alone times the CPU restatement and prints the line, the other rank
    leaves without work, no process group is formed."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "1"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["cpu_baseline"]["value"] == line["value"]
