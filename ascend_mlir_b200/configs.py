"""The five benchmark fused groups: seeded synthetic inputs, launch descriptors, algorithmic work.

Inputs are synthetic (numpy default_rng, seed 0) with the shapes, dtypes and value distributions the
benchmark configuration names; no dataset is involved.  Every group shards on its independent leading
axis: `shard(rank, world)` returns the slice of the work one GPU owns, with no data-path collective
(the gather table, the matmul B operand and the bias vectors are replicated).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np

from . import descriptors
from .descriptors import KernelSpec


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


@dataclass
class Workload:
    name: str
    spec: KernelSpec
    shape: Dict[str, int]              # shape keys of the tiling space
    inputs: List[np.ndarray]           # host tensors in kernel-argument order (bf16 as uint16 bits)
    out_shape: Tuple[int, ...]
    out_dtype: np.dtype                # uint16 for bf16
    algorithmic_bytes: int = 0         # HBM bytes one pass must move
    flops: int = 0
    bound: str = "hbm"
    units: int = 0                     # leading-axis units (rows) this workload holds
    notes: str = ""
    # (rank, world) -> Workload for that shard
    sharder: Optional[Callable[[int, int], "Workload"]] = field(default=None, repr=False)
    # generic chains: () -> the expected output (numpy, per-op rounding), for the bench's own parity check
    expected: Optional[Callable[[], np.ndarray]] = field(default=None, repr=False)

    def tiling(self, **tile_params: int) -> bytes:
        return self.spec.pack(self.shape, **tile_params)

    def new_output(self) -> np.ndarray:
        return np.zeros(self.out_shape, self.out_dtype)

    def shard(self, rank: int, world: int) -> "Workload":
        if world == 1:
            return self
        assert self.sharder is not None
        return self.sharder(rank, world)


def row_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced partition of `total` leading-axis units."""
    base, rem = divmod(total, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


# ---- config 1: out = (a + b) * b, f32 [M, N] --------------------------------------------------------------
def elementwise_chain(M: int = 4096, N: int = 4096, seed: int = 0) -> Workload:
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1.0, 1.0, (M, N)).astype(np.float32)
    b = rng.uniform(-1.0, 1.0, (M, N)).astype(np.float32)
    spec = descriptors.add_mul("f32")

    def make(a_, b_):
        m = a_.shape[0]
        w = Workload("elementwise_chain", spec, {"M": m, "N": N}, [a_, b_], (m, N), np.dtype(np.float32),
                     algorithmic_bytes=3 * m * N * 4, units=m)
        w.sharder = lambda r, k: make(*(np.ascontiguousarray(t[slice(*row_range(m, r, k))]) for t in (a_, b_)))
        return w

    return make(a, b)


# ---- config 2: split-relu-broadcast-add-mul, f16 -------------------------------------------------------------
def split_relu_broadcast_add_mul(B: int = 32, R: int = 1024, C: int = 1024, bias_axis: int = 1, seed: int = 0) -> Workload:
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((B, R, 2 * C), dtype=np.float32).astype(np.float16)
    bias = (rng.standard_normal(R if bias_axis == 1 else C, dtype=np.float32) * np.float32(0.1)).astype(np.float16)
    spec = descriptors.split_relu_bias_mul(bias_axis, "f16")

    def make(x_):
        b = x_.shape[0]
        w = Workload("split_relu_broadcast_add_mul", spec,
                     {"B": b, "R": R, "C2": 2 * C, "C": C, "BIAS": bias.shape[0]}, [x_, bias], (b, R, C),
                     np.dtype(np.float16), algorithmic_bytes=b * R * 2 * C * 2 + bias.nbytes + b * R * C * 2, units=b,
                     notes=f"bias indexed by axis {bias_axis}")
        w.sharder = lambda r, k: make(np.ascontiguousarray(x_[slice(*row_range(b, r, k))]))
        return w

    return make(x)


# ---- config 3: broadcast-add-reduce, f32 -----------------------------------------------------------------------
def broadcast_add_reduce(M: int = 8192, N: int = 8192, seed: int = 0) -> Workload:
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1.0, 1.0, (M, N)).astype(np.float32)
    b = rng.uniform(-1.0, 1.0, M).astype(np.float32)
    spec = descriptors.bcast_add_rowsum("f32")

    def make(b_, x_):
        m = x_.shape[0]
        w = Workload("broadcast_add_reduce", spec, {"M": m, "N": N}, [b_, x_], (m,), np.dtype(np.float32),
                     algorithmic_bytes=m * N * 4 + m * 4 + m * 4, units=m)
        w.sharder = lambda r, k: make(*(np.ascontiguousarray(t[slice(*row_range(m, r, k))]) for t in (b_, x_)))
        return w

    return make(b, x)


# ---- config 4: gather-elementwise fusion, bf16 -------------------------------------------------------------------
def gather_indices(rows: int, table_rows: int, dup_fraction: float, rng) -> np.ndarray:
    """`rows` int32 indices into [0, table_rows): unique draws plus ~dup_fraction copies of earlier ones, shuffled."""
    dups = int(round(rows * dup_fraction))
    uniq = min(rows - dups, table_rows)
    dups = rows - uniq
    first = rng.choice(table_rows, size=uniq, replace=False)
    extra = first[rng.integers(0, uniq, size=dups)] if dups else first[:0]
    idx = np.concatenate([first, extra])
    rng.shuffle(idx)
    return idx.astype(np.int32)


def gather_elementwise(table_rows: int = 1048576, width: int = 256, rows: int = 262144, seed: int = 0) -> Workload:
    rng = np.random.default_rng(seed)
    table = f32_to_bf16_bits(rng.standard_normal((table_rows, width), dtype=np.float32))
    idx = gather_indices(rows, table_rows, 0.05, rng)
    scale = f32_to_bf16_bits(rng.uniform(0.5, 1.5, width).astype(np.float32))
    resid = f32_to_bf16_bits(rng.standard_normal((rows, width), dtype=np.float32))
    spec = descriptors.gather_rows_scale_resid("bf16", "i32")

    def make(idx_, resid_):
        r = idx_.shape[0]
        w = Workload("gather_elementwise", spec, {"T": table_rows, "W": width, "R": r}, [table, idx_, scale, resid_],
                     (r, width), np.dtype(np.uint16),
                     algorithmic_bytes=r * 4 + r * width * 2 + width * 2 + r * width * 2 + r * width * 2, units=r,
                     notes="table replicated per GPU; each gathered row counted once")
        w.sharder = lambda rk, k: make(*(np.ascontiguousarray(t[slice(*row_range(r, rk, k))]) for t in (idx_, resid_)))
        return w

    return make(idx, resid)


# ---- config 5: matmul-add-leakyrelu, bf16 ---------------------------------------------------------------------------
def matmul_add_leakyrelu(M: int = 8192, N: int = 8192, K: int = 8192, alpha: float = 0.01, seed: int = 0) -> Workload:
    rng = np.random.default_rng(seed)
    A = f32_to_bf16_bits(rng.standard_normal((M, K), dtype=np.float32) * np.float32(0.02))
    Bm = f32_to_bf16_bits(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
    bias = f32_to_bf16_bits(rng.standard_normal(N, dtype=np.float32) * np.float32(0.1))
    spec = descriptors.matmul_bias_leakyrelu("bf16", "bf16", "bf16", alpha)

    def make(A_):
        m = A_.shape[0]
        w = Workload("matmul_add_leakyrelu", spec, {"M": m, "N": N, "K": K}, [A_, Bm, bias], (m, N), np.dtype(np.uint16),
                     algorithmic_bytes=(m * K + K * N + m * N) * 2 + N * 2, flops=2 * m * N * K, bound="tensor", units=m,
                     notes="B and bias replicated per GPU")
        w.sharder = lambda r, k: make(np.ascontiguousarray(A_[slice(*row_range(m, r, k))]))
        return w

    return make(A)


# ---- transpose-class groups (not among the five benchmark configurations; reference examples at scale) -----------
def transpose_2d(R: int = 8192, C: int = 8192, seed: int = 0) -> Workload:
    """out[c, r] = in[r, c] on f16: the standalone permutation group."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((R, C), dtype=np.float32).astype(np.float16)
    spec = descriptors.transpose_2d("f16")
    return Workload("transpose_2d", spec, {"R": R, "C": C}, [x], (C, R), np.dtype(np.float16),
                    algorithmic_bytes=2 * R * C * 2, units=C, notes="64x64 shared-memory tiles")


def relu_broadcast_transpose_add(M: int = 8192, N: int = 8192, seed: int = 0) -> Workload:
    """out[n, m] = relu(d0[m, 0]) + d1[n, m] on f16 (the reference's relu-broadcast-transpose example)."""
    rng = np.random.default_rng(seed)
    d0 = rng.standard_normal((M, 1), dtype=np.float32).astype(np.float16)
    d1 = rng.standard_normal((N, M), dtype=np.float32).astype(np.float16)
    spec = descriptors.relu_bcast_transpose_add("f16")

    def make(d1_):
        n = d1_.shape[0]
        w = Workload("relu_broadcast_transpose_add", spec, {"M": M, "N": n}, [d0, d1_], (n, M), np.dtype(np.float16),
                     algorithmic_bytes=2 * n * M * 2 + M * 2, units=n, notes="d0 replicated per GPU")
        w.sharder = lambda r, k: make(np.ascontiguousarray(d1_[slice(*row_range(n, r, k))]))
        return w

    return make(d1)


def transposed_add_mul(M: int = 8192, N: int = 8192, seed: int = 0) -> Workload:
    """out[n, m] = (a[m, n] + b[n, m]) * c[n] on f16: `a` is read through a transposed view (register blocks of 8 x 8
    elements, transposed in registers), `c` is constant along the inner dim.  Sharded by output rows: columns of `a`."""
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, N), dtype=np.float32).astype(np.float16)
    b = rng.standard_normal((N, M), dtype=np.float32).astype(np.float16)
    c = rng.standard_normal(N, dtype=np.float32).astype(np.float16)
    spec = descriptors.transposed_add_mul("f16")

    def make(a_, b_, c_):
        n = b_.shape[0]
        w = Workload("transposed_add_mul", spec, {"M": M, "N": n}, [a_, b_, c_], (n, M), np.dtype(np.float16),
                     algorithmic_bytes=3 * n * M * 2 + n * 2, units=n, notes="one operand through a transposed view")
        w.expected = lambda: ((a_.T + b_).astype(np.float16) * c_[:, None]).astype(np.float16)
        w.sharder = lambda r, k: make(np.ascontiguousarray(a_[:, slice(*row_range(n, r, k))]),
                                      np.ascontiguousarray(b_[slice(*row_range(n, r, k))]),
                                      np.ascontiguousarray(c_[slice(*row_range(n, r, k))]))
        return w

    return make(a, b, c)


# ---- generic chains: fused bodies the library has no straight-line kernel for ----------------------------------------
# They run on the kernel generated for the group (codegen/kernel_source -> NVRTC); before the generator existed
# they ran through the op-by-op interpreter at a third of the HBM roofline.
def _chain_variant(name: str, body: list, dtype: str = "f32") -> KernelSpec:
    import copy
    base = descriptors.add_mul(dtype, name=name)
    d = copy.deepcopy(base.descriptor)
    d["body"] = body
    space = copy.deepcopy(base.tiling_space)
    return KernelSpec(name=name, descriptor=d, tiling_space=space, shape_keys=dict(base.shape_keys), defaults=dict(base.defaults))


def _two_operand_chain(name: str, body: list, expected: Callable[[np.ndarray, np.ndarray], np.ndarray], M: int, N: int, seed: int) -> Workload:
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1.0, 1.0, (M, N)).astype(np.float32)
    b = rng.uniform(0.5, 1.5, (M, N)).astype(np.float32)
    spec = _chain_variant(name, body)

    def make(a_, b_):
        m = a_.shape[0]
        w = Workload(name, spec, {"M": m, "N": N}, [a_, b_], (m, N), np.dtype(np.float32), algorithmic_bytes=3 * m * N * 4, units=m,
                     notes="generated kernel (no prebuilt body matches)")
        w.expected = lambda: expected(a_, b_)
        w.sharder = lambda r, k: make(*(np.ascontiguousarray(t[slice(*row_range(m, r, k))]) for t in (a_, b_)))
        return w

    return make(a, b)


def chain_sub_div_min(M: int = 4096, N: int = 4096, seed: int = 0) -> Workload:
    """out = min((a - b) / b, a), f32, every op rounded."""
    op = descriptors.op
    return _two_operand_chain("chain_sub_div_min", [op("subf", "v0", "v1"), op("divf", "%0", "v1"), op("minimumf", "%1", "v0")],
                              lambda a, b: np.minimum((a - b) / b, a), M, N, seed)


def chain_six_ops(M: int = 4096, N: int = 4096, seed: int = 0) -> Workload:
    """r0 = a*b; out = min((max(r0 + a, 0.25) - b) * r0, 1.5), f32, every op rounded."""
    op = descriptors.op
    body = [op("mulf", "v0", "v1"), op("addf", "%0", "v0"), op("maximumf", "%1", 0.25), op("subf", "%2", "v1"),
            op("mulf", "%3", "%0"), op("minimumf", "%4", 1.5)]

    def expected(a, b):
        r0 = a * b
        return np.minimum((np.maximum(r0 + a, np.float32(0.25)) - b) * r0, np.float32(1.5))

    return _two_operand_chain("chain_six_ops", body, expected, M, N, seed)


def chain_torch_model(M: int = 4096, N: int = 4096, seed: int = 0, work_dir=None) -> Workload:
    """A torch module through the torch_e2e front (torch.export -> linalg text -> afir-opt -> afir-translate):
    out = clamp((x - shift) * scale, min=0) * y + x on f32 [M, N] with shift and scale [N] broadcast over the rows.
    Needs torch and the built front-end tools; shapes are static in the traced IR."""
    import json
    import tempfile
    from pathlib import Path

    import torch

    from .torch_e2e.pipeline import compile_model
    from .torch_e2e.tensor_spec import TensorSpec

    class GatedAffine(torch.nn.Module):
        def forward(self, x, y, scale, shift):
            return torch.clamp((x - shift) * scale, min=0.0) * y + x

    specs = [TensorSpec((M, N), torch.float32), TensorSpec((M, N), torch.float32), TensorSpec((N,), torch.float32),
             TensorSpec((N,), torch.float32)]
    root = Path(work_dir) if work_dir else Path(tempfile.mkdtemp(prefix="afir_chain_torch_model_"))
    torch.manual_seed(seed)
    built = compile_model(GatedAffine(), specs, root / "chain_torch_model", func_name="chain_torch_model")
    desc = json.loads(Path(built["kernel"]).read_text())
    space = json.loads(Path(built["space"]).read_text())
    tile_defaults = {p["name"]: p.get("default", (p.get("values") or [0])[0]) for p in space["tiling_params"] if not p.get("fixed")}
    dims = {p["name"]: p["shape_key"] for p in space["tiling_params"] if p.get("fixed")}
    spec = KernelSpec(name=desc["kernel"], descriptor=desc, tiling_space=space, shape_keys=dims, defaults=tile_defaults)
    inputs = [t.numpy() for t in built["inputs"]]
    shape = {}
    for key in dims.values():
        n, d = key[3:].split("_dim")
        shape[key] = (inputs + [np.zeros((M, N), np.float32)])[int(n)].shape[int(d)]
    w = Workload("chain_torch_model", spec, shape, inputs, (M, N), np.dtype(np.float32), algorithmic_bytes=3 * M * N * 4 + 2 * N * 4, units=M,
                 notes="torch module traced by the torch_e2e front; generated kernel")
    want = built["expected"].numpy()
    w.expected = lambda: want
    return w


GENERIC_CHAINS: Dict[str, Callable[..., Workload]] = {
    "chain_sub_div_min": chain_sub_div_min,
    "chain_six_ops": chain_six_ops,
    "chain_torch_model": chain_torch_model,
}

EXTRA_CONFIGS: Dict[str, Callable[..., Workload]] = {
    "transpose_2d": transpose_2d,
    "relu_broadcast_transpose_add": relu_broadcast_transpose_add,
    "transposed_add_mul": transposed_add_mul,
}

CONFIGS: Dict[str, Callable[..., Workload]] = {
    "elementwise_chain": elementwise_chain,
    "split_relu_broadcast_add_mul": split_relu_broadcast_add_mul,
    "broadcast_add_reduce": broadcast_add_reduce,
    "gather_elementwise": gather_elementwise,
    "matmul_add_leakyrelu": matmul_add_leakyrelu,
}
