"""Every example module through ascend_mlir_b200/examples/run_example.py: afir-opt -> afir-translate -> artifact ->
run manifest -> runtime-session --run with validation against the numpy expectation the script writes."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from ascend_mlir_b200 import build as lib_build

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
EXAMPLES = sorted(p.stem for p in (ROOT / "ascend_mlir_b200" / "examples").glob("*.mlir"))


@pytest.fixture(scope="module", autouse=True)
def built():
    lib_build.build()


def test_every_example_module_has_a_case():
    assert set(EXAMPLES) == {"elementwise_chain", "split_relu_broadcast_add_mul", "broadcast_add_reduce", "gather_elementwise",
                             "matmul_add_leakyrelu", "transpose_2d", "transposed_add", "integer_chain", "broadcast_add_reduce_scheduled"}


@pytest.mark.parametrize("name", EXAMPLES)
def test_example_runs_and_validates(name, tmp_path):
    r = subprocess.run([sys.executable, "-m", "ascend_mlir_b200.examples.run_example", name, "--out", str(tmp_path / name), "--profile"],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    lines = r.stdout.splitlines()
    assert "session.result=success" in lines and "session.validation=pass" in lines and "session.backend=cuda" in lines
    assert any(l.startswith("session.profile.score.") for l in lines)
    out = np.load(tmp_path / name / "output_0.npy")
    want = np.load(tmp_path / name / "expected_0.npy")
    assert out.shape == want.shape and out.dtype == want.dtype
