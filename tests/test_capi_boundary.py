"""The C-ABI boundary without a GPU: the library loads, exports every symbol the headers declare,
and keeps the reference's error convention (lib/CAPI/Runtime/Runtime.cpp:306-481;
test/tools/runtime/test_capi_runtime.cpp:168,176,189: the error buffer stays empty on success)."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from ascend_mlir_b200 import descriptors
from ascend_mlir_b200.runtime import CompilerError, ExecutorError, compile_kernel
from ascend_mlir_b200.runtime._capi import EXPORTS, get_lib
from ascend_mlir_b200.runtime.executor import CudaRuntime

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    names = set()
    for h in (ROOT / "include").rglob("*.h"):
        names |= set(re.findall(r"\b(afirt_[a-z_]+)\s*\(", h.read_text()))
    return names


def test_library_exports_every_declared_symbol():
    lib = get_lib()
    declared = _declared_symbols()
    assert declared, "no declarations found under include/"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(EXPORTS)
    assert b"sm_100a" in lib.afirt_runtime_version()


def test_reference_seven_entry_points_present():
    seven = ["afirt_compiler_create", "afirt_compiler_destroy", "afirt_compiler_compile", "afirt_executor_create",
             "afirt_executor_destroy", "afirt_executor_initialize", "afirt_executor_run", "afirt_executor_run_file"]
    text = (ROOT / "include" / "CAPI" / "Runtime.h").read_text()
    for name in seven:
        assert name in text and hasattr(get_lib(), name)


def _run_expect_error(rt, spec, inputs, outputs, tiling, **kw):
    with pytest.raises(ExecutorError) as e:
        rt.run(spec.binary, kw.pop("fn", spec.name), inputs, outputs, tiling, **kw)
    return str(e.value)


def test_run_before_initialize_is_an_error():
    spec = descriptors.add_mul()
    rt = CudaRuntime()
    a = np.zeros((2, 4), np.float32)
    msg = _run_expect_error(rt, spec, [a, a], [a.copy()], spec.pack({"M": 2, "N": 4}))
    assert msg == "executor has not been initialized"


def test_initialize_rejects_negative_device_and_leaves_buffer_empty_on_success():
    lib = get_lib()
    h = lib.afirt_executor_create()
    err = ctypes.create_string_buffer(256)
    assert lib.afirt_executor_initialize(ctypes.c_void_p(h), -1, err, len(err)) != 0
    assert err.value == b"device id must be non-negative"
    err = ctypes.create_string_buffer(256)
    assert lib.afirt_executor_initialize(ctypes.c_void_p(h), 0, err, len(err)) == 0
    assert err.value == b""
    lib.afirt_executor_destroy(ctypes.c_void_p(h))


def test_argument_validation_messages():
    spec = descriptors.add_mul()
    rt = CudaRuntime()
    rt.set_device(0)
    a = np.zeros((2, 4), np.float32)
    til = spec.pack({"M": 2, "N": 4})
    assert _run_expect_error(rt, spec, [a, a], [a.copy()], til, magic=0x12345678) == "unsupported kernel magic: 0x12345678"
    assert "function name is required" in _run_expect_error(rt, spec, [a, a], [a.copy()], til, fn="")
    assert "defines 'add_mul', not 'other'" in _run_expect_error(rt, spec, [a, a], [a.copy()], til, fn="other")
    assert "takes 2 inputs and 1 outputs" in _run_expect_error(rt, spec, [a], [a.copy()], til)
    assert "tiling data is 8 bytes" in _run_expect_error(rt, spec, [a, a], [a.copy()], til[:8])
    with pytest.raises(ExecutorError, match="binary data is required"):
        rt.run(b"", spec.name, [a, a], [a.copy()], til)
    with pytest.raises(ExecutorError, match="neither an AFCU container, a launch descriptor nor a kernel source"):
        rt.run(b"\x7fELF not ours", spec.name, [a, a], [a.copy()], til)


def test_error_text_is_truncated_and_terminated():
    lib = get_lib()
    h = lib.afirt_executor_create()
    err = ctypes.create_string_buffer(b"\xff" * 8, 8)
    rc = lib.afirt_executor_synchronize(ctypes.c_void_p(h), None, err, len(err))
    assert rc != 0 and err.raw[7:8] == b"\0" and err.value == b"executo"
    lib.afirt_executor_destroy(ctypes.c_void_p(h))


def test_compile_writes_container_and_manifest(tmp_path):
    spec = descriptors.bcast_add_rowsum("f32")
    src = tmp_path / "k.cuda.json"
    src.write_text(spec.descriptor_json())
    out = compile_kernel(src, tmp_path / "out", spec.name)
    blob = out.read_bytes()
    assert out.name == f"{spec.name}.bin" and blob[:4] == b"AFCU"
    # version 2: descriptor, then the group's kernel compiled for sm_100a (an ELF cubin) and its CUDA source
    json_len = int.from_bytes(blob[8:12], "little")
    assert int.from_bytes(blob[4:8], "little") == 2
    assert blob[12:12 + json_len].decode() == spec.descriptor_json()
    off = 12 + json_len
    cubin_len = int.from_bytes(blob[off:off + 4], "little")
    cubin = blob[off + 4:off + 4 + cubin_len]
    off += 4 + cubin_len
    source_len = int.from_bytes(blob[off:off + 4], "little")
    source = blob[off + 4:off + 4 + source_len].decode()
    assert off + 4 + source_len == len(blob)
    assert cubin[:4] == b"\x7fELF" and cubin_len > 1000
    # the reference's kernel signature: inputs..., outputs..., workspace, TilingData
    assert f'extern "C" __global__ void __launch_bounds__(512) {spec.name}(const void *arg0, const void *arg1, void *arg2, ' \
           "void *workspace, const __grid_constant__ TilingData t)" in source
    assert "struct TilingData {" in source and "long long SPLIT_N;" in source and "long long dim_arg1_1;" in source
    manifest = dict(line.split("=", 1) for line in (tmp_path / "out" / "manifest.txt").read_text().splitlines())
    assert manifest["kernel_name"] == spec.name and manifest["device_binary_path"] == str(out)
    assert manifest["kernel_kind"] == "vec" and manifest["soc_version"] == "sm_100a"
    assert manifest["codegen"] == "generated"
    assert (tmp_path / "out" / f"{spec.name}.cu").read_text() == source == Path(manifest["kernel_source_path"]).read_text()
    # a matmul group is the library's hand-written kernel: descriptor-only container, and the manifest says why
    mm = descriptors.matmul_bias_leakyrelu()
    mm_src = tmp_path / "mm.cuda.json"
    mm_src.write_text(mm.descriptor_json())
    mm_out = compile_kernel(mm_src, tmp_path / "out_mm", mm.name)
    mm_blob = mm_out.read_bytes()
    assert int.from_bytes(mm_blob[4:8], "little") == 1 and int.from_bytes(mm_blob[8:12], "little") == len(mm_blob) - 12
    mm_manifest = dict(line.split("=", 1) for line in (tmp_path / "out_mm" / "manifest.txt").read_text().splitlines())
    assert mm_manifest["codegen"].startswith("library") and mm_manifest["kernel_kind"] == "mix"
    # accepted reference arch names
    compile_kernel(src, tmp_path / "out2", spec.name, arch="dav-c220-vec")
    with pytest.raises(CompilerError, match="not 'wrong_name'"):
        compile_kernel(src, tmp_path / "out", "wrong_name")
    with pytest.raises(CompilerError, match="unsupported arch"):
        compile_kernel(src, tmp_path / "out", spec.name, arch="sm_90a")
    bad = tmp_path / "bad.json"
    bad.write_text('{"format": "afir-cuda-launch", "version": 1, "kernel": "x", "kernel_class": "nope"}')
    with pytest.raises(CompilerError, match="unknown kernel_class"):
        compile_kernel(bad, tmp_path / "out", "x")
    with pytest.raises(CompilerError, match="cannot open"):
        compile_kernel(tmp_path / "missing.json", tmp_path / "out", "x")


def test_descriptor_body_validation(tmp_path):
    spec = descriptors.add_mul()
    d = spec.descriptor
    for mutate, needle in [
        (lambda x: x["body"].__setitem__(0, {"op": "powf", "a": "v0", "b": "v1"}), "unsupported body op"),
        (lambda x: x["body"].__setitem__(0, {"op": "addf", "a": "v0", "b": "v7"}), "not loaded"),
        (lambda x: x["body"].__setitem__(0, {"op": "addf", "a": "%0", "b": "v1"}), "before it is defined"),
        (lambda x: x.__setitem__("arch", "sm_90a"), "sm_100a only"),
        (lambda x: x["store"].__setitem__("arg", 0), "must name an output"),
    ]:
        import copy, json
        dd = copy.deepcopy(d)
        mutate(dd)
        p = tmp_path / "m.json"
        p.write_text(json.dumps(dd))
        with pytest.raises(CompilerError, match=needle):
            compile_kernel(p, tmp_path / "o", spec.name)


def _build_c_caller(tmp_path):
    """tests/cpp/test_capi_runtime.c compiled as C99 against include/CAPI/Runtime.h and linked to the built library."""
    import subprocess
    lib_dir = ROOT / "ascend_mlir_b200" / "lib"
    exe = tmp_path / "test_capi_runtime"
    cmd = ["gcc", "-std=c99", "-O1", "-Wall", "-Wextra", "-Werror", "-ffp-contract=off", "-I", str(ROOT / "include"),
           str(ROOT / "tests" / "cpp" / "test_capi_runtime.c"), "-L", str(lib_dir), "-lAFIRRuntimeCAPI",
           f"-Wl,-rpath,{lib_dir}", "-o", str(exe)]
    built = subprocess.run(cmd, capture_output=True, text=True)
    assert built.returncode == 0, built.stderr[-3000:]
    return exe


def test_plain_c_caller_sees_the_reference_error_convention(tmp_path):
    import subprocess
    get_lib()  # makes sure the library is built
    res = subprocess.run([str(_build_c_caller(tmp_path)), "cpu"], capture_output=True, text=True)
    assert res.returncode == 0 and " passed, 0 failed" in res.stdout, res.stdout + res.stderr


@pytest.mark.gpu
def test_plain_c_caller_runs_a_kernel_and_memcmps_the_result(tmp_path):
    import subprocess
    get_lib()
    src = tmp_path / "add_mul.cuda.json"
    src.write_text(descriptors.add_mul().descriptor_json())
    res = subprocess.run([str(_build_c_caller(tmp_path)), "gpu", str(src), str(tmp_path / "artifact")], capture_output=True, text=True)
    assert res.returncode == 0 and " passed, 0 failed" in res.stdout, res.stdout + res.stderr
