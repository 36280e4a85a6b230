"""runtime-session and autotuner end to end on the GPU: manifests and tiling spaces in the reference's formats,
inputs/expected tensors as .npy, validation against the CPU oracle's outputs."""
import json
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

from ascend_mlir_b200 import build as lib_build
from ascend_mlir_b200 import configs, descriptors
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "ascend_mlir_b200" / "bin"


@pytest.fixture(scope="module", autouse=True)
def built():
    lib_build.build()


def tool(name, *args):
    return subprocess.run([str(BIN / name), *map(str, args)], capture_output=True, text=True)


def compile_artifact(tmp_path, spec, sub):
    src = tmp_path / f"{spec.name}.cuda.json"
    src.write_text(spec.descriptor_json())
    (tmp_path / f"{spec.name}.tiling_space.json").write_text(spec.tiling_space_json())
    r = tool("runtime-session", "--kernel", src, "--output", tmp_path / sub)
    assert r.returncode == 0, r.stderr
    return tmp_path / sub


def test_two_task_graph_validates_and_profiles(tmp_path):
    ew, rs = descriptors.add_mul(), descriptors.bcast_add_rowsum("f32")
    art1, art2 = compile_artifact(tmp_path, ew, "art_ew"), compile_artifact(tmp_path, rs, "art_rs")
    M, N = 300, 1024
    rng = np.random.default_rng(51)
    a = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    b = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    bias = rng.uniform(-1, 1, M).astype(np.float32)
    prod = oracle.add_mul_f32(a, b)
    sums = oracle.bcast_add_rowsum_f32(bias, prod)
    for name, arr in [("a", a), ("b", b), ("bias", bias), ("prod", prod), ("sums", sums)]:
        np.save(tmp_path / f"{name}.npy", arr)
    manifest = {"backend": "cuda", "tasks": [
        {"task_id": "chain", "artifact_root": str(art1),
         "inputs": [{"name": "a", "path": str(tmp_path / "a.npy")}, {"name": "b", "path": str(tmp_path / "b.npy")}],
         "outputs": [{"name": "out", "path": str(tmp_path / "chain_out.npy"), "shape": [M, N], "dtype": "f32"}],
         "expected_outputs": [{"name": "out", "path": str(tmp_path / "prod.npy")}],
         "tiling": {"schema": str(tmp_path / "add_mul.tiling_space.json"),
                    "params": f"CTA_THREADS=128,UNROLL=2,dim_arg0_0={M},dim_arg0_1={N}"},
         "block_dim": 0, "atol": 0.0, "rtol": 0.0, "profiling": True},
        {"task_id": "reduce", "artifact_root": str(art2), "dependencies": ["chain"],
         "inputs": [{"name": "bias", "path": str(tmp_path / "bias.npy")},
                    {"name": "x", "source": "task_output", "upstream_task": "chain", "upstream_output": "out"}],
         "outputs": [{"name": "sums", "path": str(tmp_path / "sums_out.npy")}],
         "expected_outputs": [{"name": "sums", "path": str(tmp_path / "sums.npy")}],
         "tiling": {"schema": str(tmp_path / "broadcast_add_reducesum.tiling_space.json"),
                    "params": f"CTA_THREADS=0,TEAM_LANES=0,SPLIT_N=0,BULK_COPY=1,STREAM_STAGES=0,STREAM_CHUNK=0,dim_arg0_0={M},dim_arg1_1={N}"},
         "block_dim": 0, "atol": 1e-2, "rtol": 1e-4}]}
    m = tmp_path / "run.json"
    m.write_text(json.dumps(manifest))
    r = tool("runtime-session", "--run-manifest", m, "--run")
    assert r.returncode == 0, r.stdout + r.stderr
    out = r.stdout.splitlines()
    assert "session.result=success" in out and "session.validation=pass" in out and "session.backend=cuda" in out
    assert "session.profile.count=1" in out
    assert "session.runtime.attribute.scheduler_mode=concurrent" in out and "session.runtime.counter.scheduler.task.succeeded=2" in out
    trace_path = [l.split("=", 1)[1] for l in out if l.startswith("session.profile[0]=")][0]
    trace = json.loads(Path(trace_path).read_text())
    assert trace["backend"] == "cuda" and trace["kernel_name"] == "add_mul" and trace["task_id"] == "chain"
    assert trace["score"] == trace["elapsed_us"] == trace["cycle_count"] and trace["score"] > 0
    assert trace["validation_passed"] is True and trace["inputs"][0]["shape"] == [M, N]
    assert np.array_equal(np.load(tmp_path / "chain_out.npy"), prod)
    assert np.allclose(np.load(tmp_path / "sums_out.npy"), sums, rtol=1e-4, atol=1e-2)

    # the retained copy of the profile and the session summary
    lines = dict(l.split("=", 1) for l in out if "=" in l)
    summary = json.loads(Path(lines["session.profile.summary"]).read_text())
    assert summary["tasks"][0]["task_id"] == "chain" and summary["tasks"][0]["score"] == trace["score"]
    assert Path(summary["tasks"][0]["profile_path"]) == Path(trace_path) and "/tasks/chain.json" in trace_path

    # launch tracing: arguments, alignment and named tiling words on stderr
    r = subprocess.run([str(BIN / "runtime-session"), "--run-manifest", str(m), "--run"], capture_output=True, text=True,
                       env={**os.environ, "ASCEND_RUNTIME_TRACE_LAUNCH": "1"})
    assert r.returncode == 0, r.stderr
    traced = r.stderr.splitlines()
    assert any(l.startswith("[cuda-launch] kernel=add_mul ") and "path=host" in l for l in traced)
    assert any(l.startswith("[cuda-launch] input[1] bytes=%d ptr=0x" % (M * N * 4)) and "align512=yes" in l for l in traced)
    assert f"[cuda-launch] tiling.word[2]={M} dim_arg0_0" in traced and f"[cuda-launch] tiling.word[3]={N} dim_arg0_1" in traced
    assert any(l.startswith("[cuda-launch] kernel=broadcast_add_reducesum ") for l in traced)
    # buffer samples: what the host handed over, the same bytes read back from the device, the output after its copy
    samples = [l for l in traced if "sample_hex=" in l]
    first = next(l for l in samples if l.startswith("[cuda-launch] input[0].host "))
    assert f"bytes={M * N * 4} sample_bytes=64 sample_hex=" in first and len(first.rsplit("=", 1)[1]) == 128
    back = next(l for l in samples if l.startswith("[cuda-launch] input[0].h2d_roundtrip "))
    assert back.rsplit("=", 1)[1] == first.rsplit("=", 1)[1]
    assert "[cuda-launch] input[0].h2d_roundtrip match=yes" in traced and "[cuda-launch] input[1].h2d_roundtrip match=yes" in traced
    assert any(l.startswith("[cuda-launch] output[0].host_after_d2h ") for l in samples)

    # a wrong expectation fails in the validate stage with exit code 2
    np.save(tmp_path / "prod.npy", prod + 1.0)
    r = tool("runtime-session", "--run-manifest", m, "--run")
    assert r.returncode == 2
    err = r.stderr.splitlines()
    assert "session.result=error" in err and "session.validation=fail" in err and "session.error_stage=validate" in err
    assert any("output comparison failed: max_abs_diff=1" in l for l in err)


def test_independent_tasks_run_through_the_scheduler_on_their_own_streams(tmp_path):
    """Four independent roots and one task that joins two of them: the session admits the roots together (one
    executor and stream each), every result equals the oracle's, and the serial runner gives the same files."""
    ew = descriptors.add_mul()
    art = compile_artifact(tmp_path, ew, "art_ew")
    M, N = 513, 640
    rng = np.random.default_rng(7)
    tasks, want = [], {}
    for i in range(4):
        a = rng.uniform(-1, 1, (M, N)).astype(np.float32)
        b = rng.uniform(-1, 1, (M, N)).astype(np.float32)
        np.save(tmp_path / f"a{i}.npy", a)
        np.save(tmp_path / f"b{i}.npy", b)
        want[f"root{i}"] = oracle.add_mul_f32(a, b)
        tasks.append({"task_id": f"root{i}", "artifact_root": str(art),
                      "inputs": [{"name": "a", "path": str(tmp_path / f"a{i}.npy")}, {"name": "b", "path": str(tmp_path / f"b{i}.npy")}],
                      "outputs": [{"name": "out", "path": str(tmp_path / f"root{i}_out.npy"), "shape": [M, N], "dtype": "f32"}],
                      "tiling": {"schema": str(tmp_path / "add_mul.tiling_space.json"),
                                 "params": f"CTA_THREADS=128,UNROLL=2,dim_arg0_0={M},dim_arg0_1={N}"},
                      "block_dim": 0})
    want["join"] = oracle.add_mul_f32(want["root0"], want["root1"])
    tasks.append({"task_id": "join", "artifact_root": str(art), "dependencies": ["root0", "root1"],
                  "inputs": [{"name": "a", "source": "task_output", "upstream_task": "root0", "upstream_output": "out"},
                             {"name": "b", "source": "task_output", "upstream_task": "root1", "upstream_output": "out"}],
                  "outputs": [{"name": "out", "path": str(tmp_path / "join_out.npy"), "shape": [M, N], "dtype": "f32"}],
                  "tiling": tasks[0]["tiling"], "block_dim": 0})
    m = tmp_path / "run.json"
    m.write_text(json.dumps({"backend": "cuda", "tasks": tasks}))
    r = tool("runtime-session", "--run-manifest", m, "--run")
    assert r.returncode == 0, r.stdout + r.stderr
    lines = dict(l.split("=", 1) for l in r.stdout.splitlines() if "=" in l)
    assert lines["session.runtime.attribute.scheduler_mode"] == "concurrent"
    assert lines["session.runtime.counter.scheduler.task.succeeded"] == "5"
    assert lines["session.runtime.counter.worker_count"] == "4"
    assert int(lines["session.runtime.counter.max_in_flight_tasks"]) >= 1
    for name, arr in want.items():
        assert np.array_equal(np.load(tmp_path / f"{name}_out.npy"), arr), name
        (tmp_path / f"{name}_out.npy").unlink()
    r = subprocess.run([str(BIN / "runtime-session"), "--run-manifest", str(m), "--run"], capture_output=True, text=True,
                       env={**os.environ, "ASCEND_RUNTIME_FORCE_SERIAL_SCHEDULER": "1"})
    assert r.returncode == 0 and "session.runtime.attribute.scheduler_mode=serial" in r.stdout
    for name, arr in want.items():
        assert np.array_equal(np.load(tmp_path / f"{name}_out.npy"), arr), name


def test_autotuner_searches_tile_parameters(tmp_path):
    spec = descriptors.split_relu_bias_mul(1)
    src = tmp_path / f"{spec.name}.cuda.json"
    src.write_text(spec.descriptor_json())
    space = json.loads(spec.tiling_space_json())
    space["kernel_file"] = src.name
    (tmp_path / "tiling_space.json").write_text(json.dumps(space))
    w = configs.split_relu_broadcast_add_mul(8, 256, 512, seed=52)
    np.save(tmp_path / "x.npy", w.inputs[0])
    np.save(tmp_path / "bias.npy", w.inputs[1])
    np.save(tmp_path / "expected.npy", oracle.split_relu_bias_mul_f16(w.inputs[0], w.inputs[1], 1))
    r = tool("autotuner", "--space", tmp_path / "tiling_space.json", "--inputs", f"{tmp_path / 'x.npy'},{tmp_path / 'bias.npy'}",
             "--expected", tmp_path / "expected.npy", "--shape", "B=8,R=256,C2=1024,C=512,BIAS=256", "--atol", "0", "--rtol", "0",
             "--output", tmp_path / "best_config.json")
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count(" PASS score=") == 9 and "FAIL" not in r.stdout  # 3 CTA sizes x 3 unroll depths
    best = json.loads((tmp_path / "best_config.json").read_text())
    assert best["kernel_name"] == spec.name and best["soc"] == "sm_100a"
    assert best["config"]["CTA_THREADS"] in (128, 256, 512) and best["config"]["UNROLL"] in (1, 2, 4)
    assert best["config"]["dim_arg0_2"] == 1024 and best["shape"]["C"] == 512
    assert best["best"]["score"] > 0 and best["best"]["max_abs_diff"] == 0
    assert Path(best["best"]["profile_path"]).exists()
    # a shape that contradicts the tensors is a failed candidate, not a crash
    r = tool("autotuner", "--space", tmp_path / "tiling_space.json", "--inputs", f"{tmp_path / 'x.npy'},{tmp_path / 'bias.npy'}",
             "--expected", tmp_path / "expected.npy", "--shape", "B=8,R=256,C2=1024,C=256,BIAS=256")
    assert r.returncode == 1 and "FAIL" in r.stdout and "no candidate passed validation" in r.stderr


def test_reference_style_script_runs_from_mlir_to_a_validated_result(tmp_path):
    """The stage sequence of the reference's examples/*/run.sh, stages 0 to 10, with only the tool paths changed:
    its stage names on afir-opt, `afir-translate -mlir-to-cann` writing step8_kernel.cpp, `runtime-session --kernel
    step8_kernel.cpp --kernel-kind vec` compiling that source, and a run manifest written for the reference's
    kernel -- backend "sim", a hand-kept tiling_space.json that names the schedule's tile sizes (which this target
    has no use for) beside the dims, a fixed block_dim -- executed and validated."""
    examples = ROOT / "ascend_mlir_b200" / "examples"
    stages = [[], ["--linalg-fuse-elementwise-ops"], ["--transform-interpreter", "--canonicalize", "--cse"],
              ["--one-shot-bufferize=bufferize-function-boundaries=true allow-return-allocs-from-loops=true", "--cse"],
              ["--ascendc-buffer-placement"], ["--linalg-to-ascendc", "--canonicalize", "--cse"],
              ["--ascendc-parallelize", "--canonicalize", "--cse"], ["--ascendc-prepare-for-emit", "--canonicalize", "--cse"],
              ["--canonicalize-cann-signature"]]
    src = examples / "broadcast_add_reduce_scheduled.mlir"
    for i, flags in enumerate(stages):
        dst = tmp_path / f"step{i}.mlir"
        r = tool("afir-opt", *flags, src, "-o", dst)
        assert r.returncode == 0, r.stderr
        src = dst
    kernel_cpp = tmp_path / "step8_kernel.cpp"
    r = tool("afir-translate", "-mlir-to-cann", src, "-o", kernel_cpp)
    assert r.returncode == 0, r.stderr
    name = "broadcast_add_reduce_scheduled"
    r = tool("runtime-session", "--kernel", kernel_cpp, "--kernel-kind", "vec", "--output", tmp_path / "artifact", "--name", name)
    assert r.returncode == 0, r.stderr
    manifest_txt = dict(l.split("=", 1) for l in (tmp_path / "artifact" / "manifest.txt").read_text().splitlines())
    assert manifest_txt["codegen"] == "generated"

    M, N = 640, 512
    rng = np.random.default_rng(42)
    a = rng.uniform(-1, 1, M).astype(np.float32)
    b = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    np.save(tmp_path / "input_a.npy", a)
    np.save(tmp_path / "input_b.npy", b)
    np.save(tmp_path / "output_c.npy", oracle.bcast_add_rowsum_f32(a, b))
    # the reference keeps this file by hand next to the example: tile sizes of ITS kernel, then dims under its names
    (tmp_path / "tiling_space.json").write_text(json.dumps({
        "kernel": name, "kernel_file": "step8_kernel.cpp", "soc": "Ascend910B1", "block_dim_expr": "ceil(M / TB_M)",
        "tiling_params": [{"name": "TB_M", "type": "int64", "min": 16, "max": 16, "step": 16},
                          {"name": "TB_N", "type": "int64", "values": [16]}, {"name": "Tb_M", "type": "int64", "values": [512]},
                          {"name": "dim_arg0_0", "type": "int64", "fixed": True, "shape_key": "M"},
                          {"name": "dim_arg1_1", "type": "int64", "fixed": True, "shape_key": "N"},
                          {"name": "dim_arg1_0", "type": "int64", "fixed": True, "shape_key": "M"}]}))
    run_manifest = tmp_path / "run_manifest.json"
    run_manifest.write_text(json.dumps({
        "task_id": "main", "backend": "sim", "artifact_root": str(tmp_path / "artifact"),
        "inputs": [{"name": "a", "path": str(tmp_path / "input_a.npy")}, {"name": "b", "path": str(tmp_path / "input_b.npy")}],
        "outputs": [{"name": "out", "path": str(tmp_path / "output.npy")}],
        "expected_outputs": [{"name": "out", "path": str(tmp_path / "output_c.npy")}],
        "tiling": {"schema": str(tmp_path / "tiling_space.json"),
                   "params": f"TB_M=16,TB_N=16,Tb_M=512,dim_arg0_0={M},dim_arg1_1={N},dim_arg1_0={M}"},
        "block_dim": 40, "workspace_size": 16777216, "profiling": True, "atol": 1e-3, "rtol": 1e-5}))
    r = tool("runtime-session", "--run-manifest", run_manifest, "--run")
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.splitlines()
    # a manifest written for the reference's simulator ("backend": "sim") runs on the CUDA backend: session.backend repeats
    # the name that was asked for (the reference's example scripts look for that line), session.device_backend says what ran
    assert "session.backend=sim" in lines and "session.device_backend=cuda" in lines
    assert "session.result=success" in lines and "session.validation=pass" in lines
    got = np.load(tmp_path / "output.npy")
    _, s64, abs64 = oracle.bcast_add_rowsum_f32(a, b, with_bounds=True)
    assert np.all(np.abs(got - s64) <= 1e-5 * abs64)
    # a dim that the manifest's schema names and its params leave out is an error that names it (a dim the schema does
    # not carry at all is read off the tensor bound to that argument: tests/test_runtime_tools.py)
    bad = json.loads(run_manifest.read_text())
    bad["tiling"]["params"] = f"TB_M=16,TB_N=16,Tb_M=512,dim_arg0_0={M},dim_arg1_0={M}"
    (tmp_path / "bad_manifest.json").write_text(json.dumps(bad))
    r = tool("runtime-session", "--run-manifest", tmp_path / "bad_manifest.json", "--run")
    assert r.returncode != 0 and "dim_arg1_1" in (r.stdout + r.stderr)
