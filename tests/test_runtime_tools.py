"""Host runtime and command-line tools without a GPU: the hand-rolled C++ checks of npy I/O, tiling packing,
comparator, task graph, run manifest and session (driver injected), and the runtime-session CLI contract
(exit codes 0/2/4 and key=value lines of the reference's tools/runtime-session)."""
import json
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

from ascend_mlir_b200 import build as lib_build
from ascend_mlir_b200 import descriptors

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "ascend_mlir_b200" / "bin"


@pytest.fixture(scope="module", autouse=True)
def built():
    lib_build.build()


@pytest.mark.parametrize("source", ["test_runtime_support", "test_scheduler"])
def test_cpp_checks(tmp_path, source):
    exe = tmp_path / source
    objs = [str(o) for o in sorted((ROOT / "ascend_mlir_b200" / "build").glob("*.o"))
            if "capi" not in o.name and "tools_" not in o.name]
    cmd = ["g++", "-std=c++17", "-O1", "-I", str(ROOT / "ascend_mlir_b200" / "csrc"), "-I", str(ROOT / "include"),
           str(ROOT / "tests" / "cpp" / f"{source}.cpp")] + objs + [
        "-L", "/usr/local/cuda/lib64", "-lcudart_static", "-ldl", "-lrt", "-lpthread", "-o", str(exe)]
    subprocess.run(cmd, check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert " passed, 0 failed" in res.stdout


def test_cpp_checks_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """The host runtime (json, npy, tiling, comparator, task graph, manifest, session, scheduler, retention, front end)
    rebuilt with -fsanitize=address,undefined and run through both C++ check programs: no report, all checks pass.
    Device code cannot be sanitized here; the CUDA objects are linked in as they are and never called."""
    csrc = ROOT / "ascend_mlir_b200" / "csrc"
    host = [csrc / f for f in ("common/json.cpp", "codegen/kernel_source.cpp", "codegen/nvrtc_compile.cpp", "codegen/embedded_headers.cpp",
                               "kernels/body_match.cpp", "execution/artifact_compiler.cpp", "execution/execution_session.cpp",
                               "execution/global_scheduler.cpp", "execution/output_comparator.cpp",
                               "execution/profile_retention.cpp", "execution/resource_scheduler.cpp",
                               "execution/run_manifest.cpp", "execution/task_graph.cpp", "front/group_analysis.cpp", "front/fused_generic.cpp",
                               "front/mlir_text.cpp", "front/shape_inference.cpp", "runtime/descriptor.cpp", "support/npy_io.cpp",
                               "support/tiling_schema.cpp")]
    objs = [str(o) for o in sorted((ROOT / "ascend_mlir_b200" / "build").glob("*.o"))
            if (o.name.startswith("kernels_") and o.name != "kernels_body_match.cpp.o")
            or o.name in ("runtime_executor.cpp.o", "runtime_launcher.cpp.o", "runtime_device_module.cpp.o", "runtime_host_staging.cpp.o")]
    env = {**os.environ, "ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "print_stacktrace=1"}
    flags = ["-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-I", str(csrc),
             "-I", str(ROOT / "include"), "-I", "/usr/local/cuda/include"]
    sources = host + [ROOT / "tests" / "cpp" / "test_runtime_support.cpp", ROOT / "tests" / "cpp" / "test_scheduler.cpp"]

    def compile_one(src):
        obj = tmp_path / (src.stem + ".san.o")
        return obj, subprocess.run(["g++", *flags, "-c", str(src), "-o", str(obj)], capture_output=True, text=True)

    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        compiled = list(pool.map(compile_one, sources))
    for obj, res in compiled:
        assert res.returncode == 0, res.stderr[-3000:]
    host_objs = [str(obj) for obj, _ in compiled[:len(host)]]
    for (obj, _), source in zip(compiled[len(host):], ("test_runtime_support", "test_scheduler")):
        exe = tmp_path / f"{source}.san"
        linked = subprocess.run(["g++", "-fsanitize=address,undefined", str(obj), *host_objs, *objs, "-L", "/usr/local/cuda/lib64",
                                 "-lcudart_static", "-ldl", "-lrt", "-lpthread", "-o", str(exe)], capture_output=True, text=True)
        if linked.returncode != 0 and "cannot find" in linked.stderr and "san" in linked.stderr:
            pytest.skip("sanitizer runtime libraries are not installed")
        assert linked.returncode == 0, linked.stderr[-3000:]
        res = subprocess.run([str(exe)], capture_output=True, text=True, env=env)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
        assert " passed, 0 failed" in res.stdout
        assert "runtime error" not in res.stderr and "AddressSanitizer" not in res.stderr and "LeakSanitizer" not in res.stderr


def run_tool(*args):
    return subprocess.run([str(BIN / "runtime-session"), *map(str, args)], capture_output=True, text=True)


def test_runtime_session_usage_errors_exit_4():
    r = run_tool()
    assert r.returncode == 4 and "Error: provide exactly one of --artifact-root or --kernel" in r.stderr
    r = run_tool("--artifact-root", "/nonexistent", "--kernel", "x")
    assert r.returncode == 4 and "provide exactly one of" in r.stderr
    r = run_tool("--run-manifest", "/nonexistent/m.json")
    assert r.returncode == 4 and "Error: cannot read run manifest: /nonexistent/m.json" in r.stderr
    r = run_tool("--help")
    assert r.returncode == 0 and "--run-manifest" in r.stdout


def test_a_dim_the_foreign_schema_lacks_is_read_off_the_bound_tensor(tmp_path):
    """A manifest written for the reference's kernel packs by field name; a dim_arg<N>_<D> it does not carry (the
    reference's kernel derives an output's extents from its inputs') is extent D of the tensor bound to argument N.
    Without a GPU the run then stops at the device stage, not at the bindings; a dim of an argument that is not bound
    at all is still a bindings error that names the field."""
    spec = descriptors.add_mul("f32")
    src = tmp_path / "add_mul.cuda.json"
    src.write_text(spec.descriptor_json())
    r = run_tool("--kernel", src, "--output", tmp_path / "artifact")
    assert r.returncode == 0, r.stderr
    M, N = 6, 16
    a = np.arange(M * N, dtype=np.float32).reshape(M, N)
    np.save(tmp_path / "a.npy", a)
    np.save(tmp_path / "b.npy", a + 1)
    np.save(tmp_path / "want.npy", (a + (a + 1)) * (a + 1))
    (tmp_path / "tiling_space.json").write_text(json.dumps({
        "kernel": "add_mul", "kernel_file": "step8_kernel.cpp", "soc": "Ascend910B1", "block_dim_expr": "ceil(M / TB_M)",
        "tiling_params": [{"name": "TB_M", "type": "int64", "values": [16]},
                          {"name": "dim_arg0_0", "type": "int64", "fixed": True, "shape_key": "M"}]}))
    manifest = {"task_id": "main", "backend": "sim", "artifact_root": str(tmp_path / "artifact"),
                "inputs": [{"name": "a", "path": str(tmp_path / "a.npy")}, {"name": "b", "path": str(tmp_path / "b.npy")}],
                "outputs": [{"name": "out", "path": str(tmp_path / "out.npy")}],
                "expected_outputs": [{"name": "out", "path": str(tmp_path / "want.npy")}],
                "tiling": {"schema": str(tmp_path / "tiling_space.json"), "params": f"TB_M=16,dim_arg0_0={M}"},   # no dim_arg0_1
                "block_dim": 0, "atol": 0.0, "rtol": 0.0}
    (tmp_path / "m.json").write_text(json.dumps(manifest))
    r = run_tool("--run-manifest", tmp_path / "m.json", "--run")
    out = r.stdout + r.stderr
    assert "session.error_stage=bindings" not in out and "missing field" not in out
    assert "session.error_stage=device" in out or "session.validation=pass" in out
    # with the second input unbound, the kernel's argument count no longer matches: still an error, and not a crash
    manifest["inputs"] = manifest["inputs"][:1]
    (tmp_path / "m1.json").write_text(json.dumps(manifest))
    r = run_tool("--run-manifest", tmp_path / "m1.json", "--run")
    assert r.returncode != 0 and "takes 2 inputs and 1 outputs, got 1 and 1" in r.stdout + r.stderr


def test_autotuner_takes_a_tiling_space_written_for_the_reference_kernel(tmp_path):
    """A hand-kept tiling_space.json of the reference's examples names that kernel's loop tile sizes beside the dims, in
    its own order.  The autotuner hands schema and named values to the session, which packs them for THIS kernel by
    field name: the candidate gets past the bindings (and stops at the device on a machine without a GPU), where bytes
    packed in the space's own order would be refused for their size."""
    spec = descriptors.add_mul("f32")
    kernel = tmp_path / "add_mul.cuda.json"
    kernel.write_text(spec.descriptor_json())
    M, N = 6, 16
    a = np.arange(M * N, dtype=np.float32).reshape(M, N)
    np.save(tmp_path / "a.npy", a)
    np.save(tmp_path / "b.npy", a + 1)
    np.save(tmp_path / "want.npy", (a + (a + 1)) * (a + 1))
    (tmp_path / "tiling_space.json").write_text(json.dumps({
        "kernel": "add_mul", "kernel_file": kernel.name, "soc": "Ascend910B1", "block_dim_expr": "ceil(M / TB_M)",
        "tiling_params": [{"name": "TB_M", "type": "int64", "values": [2, 3]},
                          {"name": "dim_arg0_1", "type": "int64", "fixed": True, "shape_key": "N"},
                          {"name": "dim_arg0_0", "type": "int64", "fixed": True, "shape_key": "M"}]}))
    r = subprocess.run([str(BIN / "autotuner"), "--space", str(tmp_path / "tiling_space.json"), "--inputs",
                        f"{tmp_path / 'a.npy'},{tmp_path / 'b.npy'}", "--expected", str(tmp_path / "want.npy"), "--shape", f"M={M},N={N}",
                        "--atol", "0", "--rtol", "0", "--output", str(tmp_path / "best.json")], capture_output=True, text=True)
    out = r.stdout + r.stderr
    assert "Search space: 2 candidate(s) over 1 parameter(s)" in out and "block_dim=3" in out and "block_dim=2" in out
    assert "[cuda:bindings]" not in out, out
    assert out.count("[cuda:device]") == 2 or out.count(" PASS score=") == 2, out


def test_runtime_session_compiles_and_plans(tmp_path):
    spec = descriptors.add_mul()
    src = tmp_path / "add_mul.cuda.json"
    src.write_text(spec.descriptor_json())
    r = run_tool("--kernel", src, "--output", tmp_path / "artifact", "--task-id", "t0")
    assert r.returncode == 0, r.stderr
    lines = dict(l.split("=", 1) for l in r.stdout.splitlines())
    assert lines["artifact.kernel_name"] == "add_mul" and lines["artifact.soc"] == "sm_100a"
    assert lines["session.plan.tasks"] == "1" and lines["session.plan[0]"] == "t0"
    assert (tmp_path / "artifact" / "add_mul.bin").exists()
    # the artifact root is the resumable unit: plan again without recompiling
    r = run_tool("--artifact-root", tmp_path / "artifact")
    assert r.returncode == 0 and "session.plan[0]=main" in r.stdout
    r = run_tool("--kernel", src, "--kernel-kind", "weird")
    assert r.returncode == 4 and "unsupported kernel kind: weird" in r.stderr


def _manifest(tmp_path, tasks):
    spec = descriptors.add_mul()
    src = tmp_path / "k.cuda.json"
    src.write_text(spec.descriptor_json())
    assert run_tool("--kernel", src, "--output", tmp_path / "art").returncode == 0
    m = tmp_path / "m.json"
    m.write_text(json.dumps({"backend": "cuda", "artifact_root": str(tmp_path / "art"), "tasks": tasks}))
    return m


def test_runtime_session_graph_errors_exit_2(tmp_path):
    m = _manifest(tmp_path, [{"task_id": "a", "dependencies": ["b"]}, {"task_id": "b", "dependencies": ["a"]}])
    r = run_tool("--run-manifest", m)
    assert r.returncode == 2 and "Error: task graph contains a cycle" in r.stderr
    m = _manifest(tmp_path, [{"task_id": "a", "dependencies": ["ghost"]}])
    r = run_tool("--run-manifest", m)
    assert r.returncode == 2 and "unknown task dependency" in r.stderr
    m = _manifest(tmp_path, [{"task_id": "a"}, {"task_id": "a"}])
    r = run_tool("--run-manifest", m)
    assert r.returncode == 4 and "duplicate task id" in r.stderr


def test_runtime_session_run_with_testing_driver(tmp_path):
    m = _manifest(tmp_path, [{"task_id": "first", "outputs": [{"name": "y", "shape": [2], "dtype": "f32"}]},
                             {"task_id": "second", "dependencies": ["first"],
                              "inputs": [{"name": "x", "source": "task_output", "upstream_task": "first", "upstream_output": "y"}],
                              "outputs": [{"name": "z", "shape": [2], "dtype": "f32"}]}])
    r = run_tool("--run-manifest", m, "--run", "--testing-driver", "success")
    assert r.returncode == 0, r.stderr
    out = r.stdout.splitlines()
    assert "session.plan[0]=first" in out and "session.plan[1]=second" in out
    assert "session.backend=cuda" in out and "session.result=success" in out
    assert "session.profile.count=2" in out
    assert any(l.startswith("session.runtime.counter.planned_task_count=2") for l in out)
    r = run_tool("--run-manifest", m, "--run", "--testing-driver", "bogus")
    assert r.returncode == 4 and "unsupported testing driver: bogus" in r.stderr


def test_runtime_session_retains_profiles_and_prunes_old_sessions(tmp_path):
    """Profile artifacts are copied to <tmp>/afir-cuda-runtime-profiles/<session>/tasks/<task>.json with a
    session_summary.json beside them; both that root and the session work root keep their last 20 sessions."""
    m = _manifest(tmp_path, [{"task_id": "only", "outputs": [{"name": "y", "shape": [2], "dtype": "f32"}]}])
    env = {**os.environ, "TMPDIR": str(tmp_path / "tmp")}
    (tmp_path / "tmp").mkdir()

    def run_once():
        r = subprocess.run([str(BIN / "runtime-session"), "--run-manifest", str(m), "--run", "--testing-driver", "success"],
                           capture_output=True, text=True, env=env)
        assert r.returncode == 0, r.stderr
        return dict(l.split("=", 1) for l in r.stdout.splitlines() if "=" in l)

    lines = run_once()
    summary_path = Path(lines["session.profile.summary"])
    session = lines["session.profile.session_id"]
    assert summary_path == tmp_path / "tmp" / "afir-cuda-runtime-profiles" / session / "session_summary.json"
    kept = Path(lines["session.profile[0]"])
    assert kept == summary_path.parent / "tasks" / "only.json" and json.loads(kept.read_text())["task_id"] == "only"
    summary = json.loads(summary_path.read_text())
    assert summary["schema_version"] == 1 and summary["session_id"] == session and summary["backend"] == "cuda"
    assert summary["task_count"] == summary["successful_task_count"] == 1 and summary["failed_task_count"] == 0
    assert summary["tasks"] == [{"task_id": "only", "profile_path": str(kept), "score": 1.0, "cycle_count": 1.0}]
    assert summary["total_score"] == 1.0 and summary["runtime"]["counters"]["planned_task_count"] == 1
    assert summary["runtime"]["attributes"]["scheduler_mode"] == "serial"

    for _ in range(23):
        run_once()
    for root in ("afir-cuda-runtime-profiles", "afir-cuda-runtime"):
        sessions = [p for p in (tmp_path / "tmp" / root).iterdir() if p.is_dir()]
        assert len(sessions) == 20, root
    assert not summary_path.exists(), "the first session is the oldest and has been pruned"


def test_runtime_session_reports_binding_stage_on_missing_input(tmp_path):
    # the real CUDA driver fails in the bindings stage before touching any device
    m = _manifest(tmp_path, [{"task_id": "t", "inputs": [{"name": "a", "path": str(tmp_path / "missing.npy")}],
                              "outputs": [{"name": "y", "shape": [2], "dtype": "f32"}]}])
    r = run_tool("--run-manifest", m, "--run")
    assert r.returncode == 2
    err = r.stderr.splitlines()
    assert "session.result=error" in err and "session.error_stage=bindings" in err
    assert any(l.startswith("session.error=Cannot open:") for l in err)
