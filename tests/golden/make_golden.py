#!/usr/bin/env python3
"""Regenerate the golden fixtures in this directory.

Runs the reference project's own numpy golden generators
(examples/<group>/gen_data.py or gen_inputs.py) UNCHANGED, through their
command-line flags only, and packs what they write into one .npz per group.
The reference tree is needed only to run this script; the tests read the
committed .npz files and never touch the reference.

usage: python tests/golden/make_golden.py --reference <path-to-Ascend-MLIR>
"""
import argparse
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

# name -> (example dir, script, argv, files to keep)
GROUPS = {
    # default reference shapes (128x256x128, seed 42); expected max_abs_diff == 0
    "matmul_add_leakyrelu": ("matmul-add-leakyrelu", "gen_data.py", ["--out-dir", "{out}"],
                             ["input_a", "input_b", "input_bias", "output"]),
    # default reference shapes (16x640 -> 128)
    "gather_elementwise_fusion": ("gather-elementwise-fusion", "gen_data.py", ["--out-dir", "{out}"],
                                  ["input_data", "input_indices", "input_bias", "output_out"]),
    # reduced through the scripts' own flags to keep the fixtures small
    "broadcast_add_reduce": ("broadcast-add-reduce", "gen_data.py",
                             ["--m", "96", "--n", "512", "--out-dir", "{out}"],
                             ["input_a", "input_b", "output_c"]),
    "split_relu_brc_add_mul": ("split-relu-brc-add-mul", "gen_data.py",
                               ["--M", "128", "--N", "256", "--outdir", "{out}"],
                               ["input_a", "bias0", "bias1", "scale0", "scale1", "output"]),
    "relu_broadcast_transpose": ("relu-broadcast-transpose", "gen_inputs.py",
                                 ["--m", "128", "--n", "100", "--out-dir", "{out}"],
                                 ["input_data0", "input_data1", "output_expected"]),
    "add_broadcast_concat": ("add-broadcast-concat", "gen_inputs.py",
                             ["--M", "64", "--N", "100", "--outdir", "{out}"],
                             ["input_a", "input_b", "input_c", "input_d", "output"]),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    ref = Path(args.reference)
    for name, (exdir, script, argv, keep) in GROUPS.items():
        with tempfile.TemporaryDirectory() as tmp:
            cmd = [sys.executable, str(ref / "examples" / exdir / script)] + [a.format(out=tmp) for a in argv]
            subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)
            arrays = {k: np.load(Path(tmp) / f"{k}.npy") for k in keep}
        np.savez_compressed(HERE / f"{name}.npz", **arrays)
        print(name, {k: (v.shape, str(v.dtype)) for k, v in arrays.items()})


if __name__ == "__main__":
    main()
