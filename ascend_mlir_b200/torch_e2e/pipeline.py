"""`torch_e2e_test`: a pytest decorator that takes a torch module from tracing to a verified kernel run.

Same stages and pass criterion as the reference's python/torch/framework/pipeline.py:31-120:

  0   torch -> linalg MLIR (torch2linalg.torch_to_linalg)            step0_linalg.mlir
  1-7 afir-opt passes, one file per stage                             step1_*.mlir .. step7_groups.mlir
  8   afir-translate -mlir-to-cuda                                    step8_kernel.cuda.json + .tiling_space.json
  9   eager PyTorch on the CPU gives the expected output              input_<i>.npy, expected_0.npy
  10  autotuner: compile, run every tiling candidate on the GPU, check each against the expectation

The decorated test passes when the autotuner exits 0.  Work files go to `$AFIR_TORCH_E2E_OUTPUT/<test name>`
(default `./output/torch_e2e/<test name>`), recreated on every run.  Stages 0-9 need no GPU; `compile_model`
runs just those.
"""
import functools
import json
import os
import shutil
import subprocess
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .tensor_spec import TensorSpec
from .torch2linalg import torch_to_linalg_with_state

PACKAGE_ROOT = Path(__file__).resolve().parent.parent
AFIR_OPT_STAGES = [
    ("step0b_folded.mlir", ["--linalg-fold-unit-extent-dims"]),
    ("step1_fused.mlir", ["--linalg-fuse-elementwise-ops"]),
    ("step2_shapes.mlir", ["--afir-shape-inference", "--canonicalize", "--cse"]),
    ("step3_marked.mlir", ["--mark-structured-ops"]),
    ("step4_gather.mlir", ["--fuse-gather-elementwise"]),
    ("step5_kind.mlir", ["--annotate-ascendc-kernel-kind"]),
    ("step6_matmul.mlir", ["--annotate-mix-matmul-semantics"]),
    ("step7_groups.mlir", ["--convert-afir-to-cuda"]),
]


class PipelineError(RuntimeError):
    pass


def output_root() -> Path:
    return Path(os.environ.get("AFIR_TORCH_E2E_OUTPUT", Path.cwd() / "output" / "torch_e2e"))


def find_tool(name: str) -> str:
    """PATH first, then the package's own bin directory (built by ascend_mlir_b200.build)."""
    found = shutil.which(name)
    if found:
        return found
    local = PACKAGE_ROOT / "bin" / name
    if local.exists():
        return str(local)
    raise PipelineError(f"tool '{name}' not found on PATH or in {PACKAGE_ROOT / 'bin'}; run ascend_mlir_b200.build.build()")


def _run(cmd: Sequence[str], what: str) -> subprocess.CompletedProcess:
    proc = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if proc.returncode != 0:
        raise PipelineError(f"{what} failed (exit {proc.returncode}): {' '.join(map(str, cmd))}\n{proc.stdout[-2000:]}{proc.stderr[-2000:]}")
    return proc


def save_tensor(path: Path, t: torch.Tensor) -> None:
    """.npy as the runtime reads it; bfloat16 (which numpy lacks) as 2-byte opaque items."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        np.save(path, t.view(torch.int16).numpy().view(np.dtype("V2")))
    else:
        np.save(path, t.numpy())


def run_mlir_pipeline(work_dir: Path) -> Path:
    """Stages 1-8 on `work_dir/step0_linalg.mlir`; returns the launch descriptor path."""
    src = work_dir / "step0_linalg.mlir"
    if not src.exists():
        raise PipelineError(f"missing {src}")
    afir_opt, afir_translate = find_tool("afir-opt"), find_tool("afir-translate")
    for out_name, passes in AFIR_OPT_STAGES:
        dst = work_dir / out_name
        _run([afir_opt, *passes, src, "-o", dst], f"afir-opt {' '.join(passes)}")
        src = dst
    kernel = work_dir / "step8_kernel.cuda.json"
    _run([afir_translate, "-mlir-to-cuda", src, "-o", kernel, "--tiling-space-out", work_dir / "step8_kernel.tiling_space.json"],
         "afir-translate -mlir-to-cuda")
    return kernel


def patch_tiling_space(path: Path) -> None:
    """Search parameters that came without candidates get their default as the only candidate, so that the
    autotuner always has a complete grid (the reference patches its spaces the same way, pipeline.py:131-162)."""
    space = json.loads(path.read_text())
    changed = False
    for p in space.get("tiling_params", []):
        if p.get("fixed") or p.get("values") or "min" in p:
            continue
        p["values"] = [p.get("default", p.get("value", 0))]
        changed = True
    if changed:
        path.write_text(json.dumps(space, indent=2) + "\n")


def build_shape_string(tiling_space_path: Path, inputs: Sequence[torch.Tensor]) -> str:
    """`--shape` for the autotuner: every fixed parameter's shape_key ("arg<N>_dim<D>") looked up in the inputs."""
    space = json.loads(tiling_space_path.read_text())
    parts = []
    for p in space.get("tiling_params", []):
        key = p.get("shape_key")
        if not p.get("fixed") or not key:
            continue
        arg, dim = key.split("_")
        parts.append(f"{key}={inputs[int(arg[3:])].shape[int(dim[3:])]}")
    return ",".join(parts)


def compile_model(model: torch.nn.Module, specs: Sequence[TensorSpec], work_dir: Path,
                  verify_shapes: Optional[Dict[str, int]] = None, func_name: str = "forward") -> Dict[str, object]:
    """Stages 0-9.  Returns the paths and tensors stage 10 needs."""
    if work_dir.exists():
        shutil.rmtree(work_dir)
    work_dir.mkdir(parents=True)
    pool: Dict[str, object] = {}
    per_input = [spec.dynamic_dims(pool) for spec in specs]
    dynamic_shapes = tuple(d or None for d in per_input) if any(per_input) else None
    trace_inputs = [spec.make_sample() for spec in specs]
    # parameters and buffers of the model become kernel arguments after the user inputs
    text, state = torch_to_linalg_with_state(model, trace_inputs, dynamic_shapes, func_name=func_name)
    (work_dir / "step0_linalg.mlir").write_text(text)
    kernel = run_mlir_pipeline(work_dir)
    space = work_dir / "step8_kernel.tiling_space.json"
    patch_tiling_space(space)

    user_inputs = [spec.make_sample(verify_shapes or {}) for spec in specs]
    with torch.no_grad():
        expected = model.eval()(*user_inputs)
    verify_inputs = user_inputs + [t for _, t in state]
    for i, t in enumerate(verify_inputs):
        save_tensor(work_dir / f"input_{i}.npy", t)
    save_tensor(work_dir / "expected_0.npy", expected)
    return {"kernel": kernel, "space": space, "inputs": verify_inputs, "expected": expected, "state": [n for n, _ in state],
            "num_inputs": len(verify_inputs), "shape": build_shape_string(space, verify_inputs)}


def run_autotuner(work_dir: Path, num_inputs: int, shape: str, atol: float = 1.0, rtol: float = 1e-2) -> Dict[str, object]:
    """Stage 10.  Raises PipelineError unless the autotuner exits 0; returns the best configuration it wrote."""
    cmd = [find_tool("autotuner"), "--space", work_dir / "step8_kernel.tiling_space.json", "--kernel", work_dir / "step8_kernel.cuda.json",
           "--inputs", ",".join(str(work_dir / f"input_{i}.npy") for i in range(num_inputs)),
           "--expected", work_dir / "expected_0.npy", "--output", work_dir / "best_config.json",
           "--atol", repr(atol), "--rtol", repr(rtol)]
    cmd += [f"--shape={shape}"]  # required by the tool even when every dim is static (then it is empty)
    proc = _run(cmd, "autotuner")
    (work_dir / "autotuner.log").write_text(proc.stdout + proc.stderr)
    return json.loads((work_dir / "best_config.json").read_text())


def torch_e2e_test(func=None, *, verify_shapes: Optional[Dict[str, int]] = None, atol: float = 1.0, rtol: float = 1e-2):
    """Decorator: the function returns `(model, [TensorSpec, ...])`; the wrapper runs stages 0-10.

    `verify_shapes` gives the sizes of named dynamic dimensions for the verification run (others are 64).
    Usable bare (`@torch_e2e_test`) or with arguments, like the reference's decorator.
    """
    def decorate(fn):
        @functools.wraps(fn)
        def wrapper():
            model, specs = fn()
            work_dir = output_root() / fn.__name__
            built = compile_model(model, specs, work_dir, verify_shapes)
            best = run_autotuner(work_dir, built["num_inputs"], built["shape"], atol, rtol)
            print(f"torch_e2e {fn.__name__}: best {best.get('config')} score {best.get('best', {}).get('score')} us")
            return None
        return wrapper
    return decorate(func) if func is not None else decorate
