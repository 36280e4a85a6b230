"""The reference's own unit tests of its Python TilingSchema (python/test/test_tiling_schema.py), run against this
repository's mirror of that class and, beside it, against the reference's class: the two must pass and fail the same
cases.  Needs a reference checkout (AFIR_REFERENCE_EXAMPLES names its examples/ directory); skipped otherwise."""
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
EXAMPLES = Path(os.environ["AFIR_REFERENCE_EXAMPLES"]) if os.environ.get("AFIR_REFERENCE_EXAMPLES") else None

pytestmark = pytest.mark.skipif(EXAMPLES is None or not (EXAMPLES.parent / "python" / "test" / "test_tiling_schema.py").exists(),
                                reason="AFIR_REFERENCE_EXAMPLES does not name the examples/ directory of a reference checkout")


def outcomes(cwd, env):
    r = subprocess.run([sys.executable, "-m", "pytest", "-p", "no:cacheprovider", "-q", "-rA", "python/test/test_tiling_schema.py"],
                       cwd=cwd, env=env, capture_output=True, text=True, timeout=300)
    found = dict((m.group(2), m.group(1)) for m in re.finditer(r"^(PASSED|FAILED) \S*::(\w+)", r.stdout, re.M))
    assert found, r.stdout[-2000:] + r.stderr[-2000:]
    return found


def test_tiling_schema_mirror_passes_what_the_reference_class_passes(tmp_path):
    checkout = EXAMPLES.parent
    # a tree shaped like the reference's, whose python/runtime/tiling_schema.py is this repository's class
    mine = tmp_path / "mine"
    (mine / "python" / "runtime").mkdir(parents=True)
    (mine / "python" / "test").mkdir()
    (mine / "examples" / "broadcast-add-reduce").mkdir(parents=True)
    (mine / "python" / "__init__.py").write_text("")
    (mine / "python" / "runtime" / "__init__.py").write_text("")
    (mine / "python" / "runtime" / "tiling_schema.py").write_text("from ascend_mlir_b200.runtime.tiling_schema import *  # noqa: F401,F403\n")
    shutil.copy(checkout / "python" / "test" / "test_tiling_schema.py", mine / "python" / "test")
    shutil.copy(EXAMPLES / "broadcast-add-reduce" / "tiling_space.json", mine / "examples" / "broadcast-add-reduce")
    # and the same test file beside the reference's own class
    theirs = tmp_path / "theirs"
    (theirs / "python" / "runtime").mkdir(parents=True)
    (theirs / "python" / "test").mkdir()
    (theirs / "examples" / "broadcast-add-reduce").mkdir(parents=True)
    (theirs / "python" / "__init__.py").write_text("")
    (theirs / "python" / "runtime" / "__init__.py").write_text("")
    shutil.copy(checkout / "python" / "runtime" / "tiling_schema.py", theirs / "python" / "runtime")
    shutil.copy(checkout / "python" / "test" / "test_tiling_schema.py", theirs / "python" / "test")
    shutil.copy(EXAMPLES / "broadcast-add-reduce" / "tiling_space.json", theirs / "examples" / "broadcast-add-reduce")
    env = {**os.environ, "PYTHONPATH": str(ROOT)}
    got, want = outcomes(mine, env), outcomes(theirs, env)
    assert got == want
    # (two cases fail on both sides: the example's tiling_space.json gained a field, Tb_M, after the test was written)
    assert sum(v == "PASSED" for v in got.values()) >= 10


def test_the_reference_binding_drives_this_library_unmodified(tmp_path):
    """python/runtime/{compiler,executor}.py of the reference, imported as they are with AFIRT_CAPI_LIB naming this
    repository's libAFIRRuntimeCAPI.so: BishengCompiler.compile_and_link compiles a descriptor to a container, a missing
    source is a CompilerError carrying the library's text, AscendRuntime() creates an executor, and running before
    set_device fails with the reference's own message.  (Launching needs a GPU: tests/test_capi_boundary.py and the GPU
    suite cover afirt_executor_run through this repository's mirror of the same binding.)"""
    from ascend_mlir_b200 import build as lib_build
    lib = lib_build.build()
    script = tmp_path / "drive.py"
    script.write_text(f"""
import json, pathlib, sys
sys.path.insert(0, {str(EXAMPLES.parent / 'python')!r})
sys.path.insert(0, {str(ROOT)!r})
import numpy as np
from runtime.compiler import BishengCompiler, CompilerError
from runtime.executor import AscendRuntime, ExecutorError
from ascend_mlir_b200 import descriptors
tmp = pathlib.Path({str(tmp_path)!r})
spec = descriptors.add_mul("f32")
src = tmp / "add_mul.cuda.json"
src.write_text(spec.descriptor_json())
compiler = BishengCompiler(ascend_root=tmp, soc_version="Ascend910B1")
out = compiler.compile_and_link(src, tmp / "out", "add_mul")
result = {{"container": out.read_bytes()[:4].decode(), "name": out.name}}
try:
    compiler.compile_and_link(tmp / "missing.cpp", tmp / "out2", "x")
except CompilerError as e:
    result["missing"] = str(e)
rt = AscendRuntime(ascend_root=tmp, soc_version="Ascend910B1")
try:
    rt.run(out.read_bytes(), "add_mul", [np.zeros((2, 4), np.float32)] * 2, [np.zeros((2, 4), np.float32)], spec.pack({{"M": 2, "N": 4}}), 1)
except ExecutorError as e:
    result["uninitialized"] = str(e)
print("RESULT " + json.dumps(result))
""")
    env = {**os.environ, "AFIRT_CAPI_LIB": str(lib)}
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    import json
    result = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][0][7:])
    assert result["container"] == "AFCU" and result["name"] == "add_mul.bin"
    assert result["missing"].startswith("cannot open ") and result["missing"].endswith("missing.cpp")
    assert result["uninitialized"] == "executor has not been initialized"
