#!/usr/bin/env python3
"""One example from MLIR text to a validated run, the flow of the reference's examples/*/run.sh:

    python -m ascend_mlir_b200.examples.run_example broadcast_add_reduce [--out DIR] [--profile]

  step 1-7  afir-opt          <name>.mlir -> step7_groups.mlir     (mark, fuse, classify, convert)
  step 8    afir-translate    -> kernel.cuda.json + tiling_space.json
  step 9    numpy             inputs and the expected output as .npy   (the reference runs gen_data.py here)
  step 10   runtime-session   --kernel: artifact directory with manifest.txt and <name>.bin
  step 11   runtime-session   --run-manifest run_manifest.json --run: launch, compare, session.* lines

The expectation is computed here with numpy in the element type of the group (numpy rounds after every
float16 operation, as the IR does); bf16 groups are computed in float32 and compared with the reference's
example tolerances.  Exit code = runtime-session's (0 ok, 2 run or validation failed, 4 usage).
"""
import argparse
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
BIN = HERE.parent / "bin"
PASSES = ["--afir-shape-inference", "--linalg-fuse-elementwise-ops", "--mark-structured-ops", "--fuse-gather-elementwise",
          "--annotate-ascendc-kernel-kind", "--annotate-mix-matmul-semantics", "--convert-afir-to-cuda"]


def bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 storage (round to nearest even) as 2-byte opaque items, the way the runtime reads .npy."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16).view(np.dtype("V2"))


def bf16_to_f32(v: np.ndarray) -> np.ndarray:
    return (v.view(np.uint16).astype(np.uint32) << 16).view(np.float32)


def make_case(name: str, rng):
    """(inputs in argument order, expected output, atol, rtol) at the example's own small shape."""
    if name == "elementwise_chain":  # static [4096, 4096] in the MLIR
        a = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
        b = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
        return [a, b], ((a + b) * b).astype(np.float32), 0.0, 0.0
    if name == "split_relu_broadcast_add_mul":  # static [32, 1024, 2048]
        x = rng.standard_normal((32, 1024, 2048), dtype=np.float32).astype(np.float16)
        bias = (rng.standard_normal(1024, dtype=np.float32) * np.float32(0.1)).astype(np.float16)
        h0, h1 = x[..., :1024], x[..., 1024:]
        want = ((np.maximum(h0, np.float16(0)) + bias[None, :, None]).astype(np.float16) * h1).astype(np.float16)
        return [x, bias], want, 0.0, 0.0
    if name in ("broadcast_add_reduce", "broadcast_add_reduce_scheduled"):  # the second: already fused, with a tiling schedule beside it
        b = rng.uniform(-1, 1, 640).astype(np.float32)
        x = rng.uniform(-1, 1, (640, 512)).astype(np.float32)
        return [b, x], (b[:, None].astype(np.float64) + x).sum(axis=1).astype(np.float32), 1e-3, 1e-5
    if name == "gather_elementwise":
        table = rng.standard_normal((4096, 256), dtype=np.float32)
        idx = rng.integers(0, 4096, 1000).astype(np.int32)
        scale = rng.uniform(0.5, 1.5, 256).astype(np.float32)
        resid = rng.standard_normal((1000, 256), dtype=np.float32)
        tb, sb, rb = bf16(table), bf16(scale), bf16(resid)
        prod = bf16_to_f32(bf16(bf16_to_f32(tb)[idx] * bf16_to_f32(sb)[None, :]))
        return [tb, idx, sb, rb], bf16(prod + bf16_to_f32(rb)), 1e-2, 1e-2
    if name == "matmul_add_leakyrelu":
        A = bf16(rng.standard_normal((384, 320), dtype=np.float32) * np.float32(0.1))
        B = bf16(rng.standard_normal((320, 512), dtype=np.float32) * np.float32(0.1))
        bias = bf16(rng.standard_normal(512, dtype=np.float32) * np.float32(0.1))
        x = bf16_to_f32(A).astype(np.float64) @ bf16_to_f32(B).astype(np.float64) + bf16_to_f32(bias)[None, :]
        return [A, B, bias], bf16(np.maximum(x, 0.01 * x).astype(np.float32)), 1e-2, 1e-2
    if name == "integer_chain":
        a = rng.integers(-32768, 32767, (333, 1000), endpoint=True).astype(np.int16)
        b = rng.integers(-32768, 32767, 1000, endpoint=True).astype(np.int16)
        with np.errstate(over="ignore"):
            want = ((a + b[None, :]).astype(np.int16) * a).astype(np.int16)
        return [a, b], want, 0.0, 0.0
    if name == "transpose_2d":
        x = rng.standard_normal((1000, 520)).astype(np.float16)
        return [x], np.ascontiguousarray(x.T), 0.0, 0.0
    if name == "transposed_add":
        a = rng.standard_normal((520, 264)).astype(np.float16)
        b = rng.standard_normal((264, 520)).astype(np.float16)
        return [a, b], (a.T + b).astype(np.float16), 0.0, 0.0
    raise SystemExit(f"unknown example '{name}'; have: " + ", ".join(sorted(p.stem for p in HERE.glob("*.mlir"))))


def run(cmd, **kw):
    print("+ " + " ".join(str(c) for c in cmd), flush=True)
    return subprocess.run([str(c) for c in cmd], **kw)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("example", help="name of an .mlir file in this directory, without the suffix")
    ap.add_argument("--out", default=None, help="work directory (default: ./out_<example>)")
    ap.add_argument("--profile", action="store_true", help="ask the session for a kernel-time profile")
    ap.add_argument("--seed", type=int, default=42)
    args = ap.parse_args()
    src = HERE / f"{args.example}.mlir"
    if not src.exists():
        make_case(args.example, None)
    out = Path(args.out or f"out_{args.example}").resolve()
    out.mkdir(parents=True, exist_ok=True)

    for tool in ("afir-opt", "afir-translate", "runtime-session"):
        if not (BIN / tool).exists():
            raise SystemExit(f"{BIN / tool} is missing: build first (python -m ascend_mlir_b200.build)")
    if run([BIN / "afir-opt", *PASSES, src, "-o", out / "step7_groups.mlir"]).returncode:
        return 4
    if run([BIN / "afir-translate", "-mlir-to-cuda", out / "step7_groups.mlir", "-o", out / "kernel.cuda.json",
            "--tiling-space-out", out / "tiling_space.json"]).returncode:
        return 4

    inputs, expected, atol, rtol = make_case(args.example, np.random.default_rng(args.seed))
    arrays = inputs + [expected]
    for i, a in enumerate(inputs):
        np.save(out / f"input_{i}.npy", a)
    np.save(out / "expected_0.npy", expected)

    space = json.loads((out / "tiling_space.json").read_text())
    kernel = space["kernel"]
    params = []
    for p in space["tiling_params"]:
        if p.get("fixed"):
            arg, dim = p["shape_key"][3:].split("_dim")
            params.append(f"{p['name']}={arrays[int(arg)].shape[int(dim)]}")
        else:
            params.append(f"{p['name']}={p['default']}")
    if run([BIN / "runtime-session", f"--kernel={out / 'kernel.cuda.json'}", f"--output={out / 'artifact'}", f"--name={kernel}"]).returncode:
        return 4
    manifest = {"backend": "cuda", "artifact_root": str(out / "artifact"), "task_id": args.example,
                "inputs": [{"name": f"in{i}", "path": str(out / f"input_{i}.npy")} for i in range(len(inputs))],
                "outputs": [{"name": "out", "path": str(out / "output_0.npy")}],
                "expected_outputs": [{"name": "out", "path": str(out / "expected_0.npy")}],
                "tiling": {"schema": str(out / "tiling_space.json"), "params": ",".join(params)},
                "block_dim": 0, "profiling": bool(args.profile), "atol": atol, "rtol": rtol}
    (out / "run_manifest.json").write_text(json.dumps(manifest, indent=2) + "\n")
    return run([BIN / "runtime-session", f"--run-manifest={out / 'run_manifest.json'}", "--run"]).returncode


if __name__ == "__main__":
    sys.exit(main())
