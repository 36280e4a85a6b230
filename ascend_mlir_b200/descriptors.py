"""Launch descriptors and tiling spaces for the fused-group classes.

A launch descriptor is what the translate step emits for one fused kernel (the counterpart of the
reference's generated step8_kernel.cpp) and `tiling_space.json` keeps the reference's schema
(lib/Target/CannKernel/CannTranslation.cpp:1987-2042): {kernel, kernel_file, soc, block_dim_expr,
tiling_params:[{name, type, fixed, shape_key | values | min/max/step | value}]}.  TilingData is the
reference's all-int64 struct: tile parameters first, then dim_arg<N>_<D> for every dynamic dim
(lib/Conversion/AscendCPrepareForEmit/AscendCPrepareForEmitPass.cpp:200-216).

The builders below write the descriptors of the groups this repository benchmarks and of the
reference's six examples; any other fused elementwise / reduce / gather group is expressed with the
same vocabulary (domain, loads, store, body).
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .runtime.tiling_schema import TilingSchema

FORMAT = "afir-cuda-launch"
SOC = "sm_100a"


def op(name: str, a, b) -> dict:
    return {"op": name, "a": a, "b": b}


def container(descriptor: dict) -> bytes:
    """Seal a descriptor into the .bin container (what afirt_compiler_compile writes)."""
    text = json.dumps(descriptor, separators=(",", ":")).encode()
    return b"AFCU" + struct.pack("<II", 1, len(text)) + text


@dataclass
class KernelSpec:
    name: str
    descriptor: dict
    tiling_space: dict
    shape_keys: Dict[str, str] = field(default_factory=dict)  # tiling field -> shape key
    defaults: Dict[str, int] = field(default_factory=dict)    # tile-parameter defaults
    magic: int = 0x41415246

    def __post_init__(self):
        self.binary = container(self.descriptor)
        self.schema = TilingSchema.from_dict(self.tiling_space, self.name)

    def pack(self, shape: Dict[str, int], **tile_params: int) -> bytes:
        values = dict(self.defaults)
        values.update(tile_params)
        for fname, key in self.shape_keys.items():
            values[fname] = shape[key]
        return self.schema.pack(**values)

    def descriptor_json(self) -> str:
        return json.dumps(self.descriptor, indent=2)

    def tiling_space_json(self) -> str:
        return json.dumps(self.tiling_space, indent=2)


def _spec(name, kernel_class, dtype, num_inputs, num_outputs, tile_params, dims, body_fields, launch,
          block_dim_expr="0", magic=0x41415246) -> KernelSpec:
    """tile_params: [(name, default, values)], dims: [(field, shape_key)]."""
    tiling_names = [p[0] for p in tile_params] + [d[0] for d in dims]
    desc = {"format": FORMAT, "version": 1, "kernel": name, "kernel_class": kernel_class, "arch": SOC, "dtype": dtype,
            "num_inputs": num_inputs, "num_outputs": num_outputs,
            "tiling": [{"name": n, "type": "int64"} for n in tiling_names], "launch": launch}
    desc.update(body_fields)
    params = []
    for pname, default, values in tile_params:
        params.append({"name": pname, "type": "int64", "values": list(values), "default": default})
    for fname, key in dims:
        params.append({"name": fname, "type": "int64", "fixed": True, "shape_key": key})
    space = {"kernel": name, "kernel_file": f"{name}.cuda.json", "soc": SOC, "block_dim_expr": block_dim_expr,
             "tiling_params": params}
    return KernelSpec(name=name, descriptor=desc, tiling_space=space, shape_keys=dict(dims),
                      defaults={p[0]: p[1] for p in tile_params}, magic=magic)


_EW_TILE = [("CTA_THREADS", 128, (128, 256, 512)), ("UNROLL", 2, (1, 2, 4))]
_GATHER_TILE = [("CTA_THREADS", 128, (128, 256, 512)), ("UNROLL", 1, (1, 2, 4)), ("BULK_COPY", 0, (0, 1)),
                ("STREAM_STAGES", 0, (0, 2, 3, 4, 6)), ("STREAM_ROWS", 0, (0, 2, 4, 8, 16)),
                ("STREAM_WARPS", 0, (0, 4, 8, 16))]
_GATHER_LAUNCH = {"cta_threads": "CTA_THREADS", "unroll": "UNROLL", "bulk_copy": "BULK_COPY",
                  "stream_stages": "STREAM_STAGES", "stream_rows": "STREAM_ROWS",
                  "stream_warps": "STREAM_WARPS"}
_EW_LAUNCH = {"cta_threads": "CTA_THREADS", "unroll": "UNROLL"}


# ---- elementwise / broadcast / split / concat ------------------------------------------------------
def add_mul(dtype: str = "f32", name: str = "add_mul") -> KernelSpec:
    """out = (a + b) * b on [M, N] (afir.add then afir.mul)."""
    dims = [("dim_arg0_0", "M"), ("dim_arg0_1", "N")]
    shp = ["dim_arg0_0", "dim_arg0_1"]
    view = lambda arg: {"arg": arg, "shape": shp, "map": [0, 1]}  # noqa: E731
    body = {"domain": shp, "loads": [view(0), view(1)], "store": view(2),
            "body": [op("addf", "v0", "v1"), op("mulf", "%0", "v1")]}
    return _spec(name, "elementwise", dtype, 2, 1, _EW_TILE, dims, body, _EW_LAUNCH)


def split_relu_bias_mul(bias_axis: int = 1, dtype: str = "f16", name: str = "split_relu_broadcast_add_mul") -> KernelSpec:
    """x[B,R,2C] split on the last axis into h0,h1; out[B,R,C] = (relu(h0) + bias) * h1.

    bias_axis 1: bias[R] follows the row (the reference example's row map); 2: bias[C] follows the column.
    """
    dims = [("dim_arg0_0", "B"), ("dim_arg0_1", "R"), ("dim_arg0_2", "C2"), ("dim_arg2_2", "C"), ("dim_arg1_0", "BIAS")]
    xshape = ["dim_arg0_0", "dim_arg0_1", "dim_arg0_2"]
    oshape = ["dim_arg0_0", "dim_arg0_1", "dim_arg2_2"]
    body = {"domain": oshape,
            "loads": [{"arg": 0, "shape": xshape, "map": [0, 1, 2], "offset": [0, 0, 0]},
                      {"arg": 1, "shape": ["dim_arg1_0"], "map": [bias_axis]},
                      {"arg": 0, "shape": xshape, "map": [0, 1, 2], "offset": [0, 0, "dim_arg2_2"]}],
            "store": {"arg": 2, "shape": oshape, "map": [0, 1, 2]},
            "body": [op("maximumf", "v0", 0.0), op("addf", "%0", "v1"), op("mulf", "%1", "v2")]}
    return _spec(name, "elementwise", dtype, 2, 1, _EW_TILE, dims, body, _EW_LAUNCH)


def split_rows_relu_bias_scale(dtype: str = "f16", name: str = "ewop_broadcast_split") -> KernelSpec:
    """The reference example: rows of a[M,N] split in halves, out_h = (relu(a_h) + bias_h[m]) * scale_h[n],
    halves concatenated on axis 0 (two groups writing the two halves of one output, no copy)."""
    dims = [("dim_arg0_0", "M"), ("dim_arg0_1", "N"), ("dim_arg1_0", "HM"), ("dim_arg2_0", "HM"),
            ("dim_arg3_0", "N"), ("dim_arg4_0", "N")]
    ashape = ["dim_arg0_0", "dim_arg0_1"]
    dom = ["dim_arg1_0", "dim_arg0_1"]
    body_ops = [op("maximumf", "v0", 0.0), op("addf", "%0", "v1"), op("mulf", "%1", "v2")]

    def group(off, bias_arg, scale_arg, hm):
        return {"domain": dom,
                "loads": [{"arg": 0, "shape": ashape, "map": [0, 1], "offset": [off, 0]},
                          {"arg": bias_arg, "shape": [hm], "map": [0]},
                          {"arg": scale_arg, "shape": ["dim_arg0_1"], "map": [1]}],
                "store": {"arg": 5, "shape": ashape, "map": [0, 1], "offset": [off, 0]},
                "body": body_ops}

    body = {"groups": [group(0, 1, 3, "dim_arg1_0"), group("dim_arg1_0", 2, 4, "dim_arg2_0")]}
    return _spec(name, "elementwise", dtype, 5, 1, _EW_TILE, dims, body, _EW_LAUNCH)


def add_mul_concat(dtype: str = "f16", name: str = "ewop_broadcast_concat") -> KernelSpec:
    """The reference example: out[2M,N] = concat(a[m] + b[m,n], c[m] * d[m,n], axis 0)."""
    dims = [("dim_arg0_0", "M"), ("dim_arg1_1", "N"), ("dim_arg4_0", "M2")]
    dom = ["dim_arg0_0", "dim_arg1_1"]
    oshape = ["dim_arg4_0", "dim_arg1_1"]

    def group(vec_arg, mat_arg, opname, off):
        return {"domain": dom,
                "loads": [{"arg": vec_arg, "shape": ["dim_arg0_0"], "map": [0]},
                          {"arg": mat_arg, "shape": dom, "map": [0, 1]}],
                "store": {"arg": 4, "shape": oshape, "map": [0, 1], "offset": [off, 0]},
                "body": [op(opname, "v0", "v1")]}

    body = {"groups": [group(0, 1, "addf", 0), group(2, 3, "mulf", "dim_arg0_0")]}
    return _spec(name, "elementwise", dtype, 4, 1, _EW_TILE, dims, body, _EW_LAUNCH)


def relu_bcast_transpose_add(dtype: str = "f16", name: str = "relu_transpose_broadcast_add") -> KernelSpec:
    """The reference example: out[n,m] = relu(d0[m,0]) + d1[n,m]; d0 is read through the map (d0,d1)->(d1,0)."""
    dims = [("dim_arg0_0", "M"), ("dim_arg1_0", "N")]
    dom = ["dim_arg1_0", "dim_arg0_0"]
    body = {"domain": dom,
            "loads": [{"arg": 0, "shape": ["dim_arg0_0", 1], "map": [1, -1]},
                      {"arg": 1, "shape": dom, "map": [0, 1]}],
            "store": {"arg": 2, "shape": dom, "map": [0, 1]},
            "body": [op("maximumf", "v0", 0.0), op("addf", "%0", "v1")]}
    return _spec(name, "elementwise", dtype, 2, 1, _EW_TILE, dims, body, _EW_LAUNCH)


def transposed_add_mul(dtype: str = "f16", name: str = "transposed_add_mul") -> KernelSpec:
    """out[n, m] = (a[m, n] + b[n, m]) * c[n]: `a` is read through a transposed view, `c` is constant along the
    inner dim.  Arguments: a [M, N], b [N, M], c [N] -> out [N, M]."""
    dims = [("dim_arg0_0", "M"), ("dim_arg0_1", "N")]
    dom = ["dim_arg0_1", "dim_arg0_0"]
    body = {"domain": dom,
            "loads": [{"arg": 0, "shape": ["dim_arg0_0", "dim_arg0_1"], "map": [1, 0]},
                      {"arg": 1, "shape": dom, "map": [0, 1]},
                      {"arg": 2, "shape": ["dim_arg0_1"], "map": [0]}],
            "store": {"arg": 3, "shape": dom, "map": [0, 1]},
            "body": [op("addf", "v0", "v1"), op("mulf", "%0", "v2")]}
    return _spec(name, "elementwise", dtype, 3, 1, _EW_TILE, dims, body, _EW_LAUNCH)


def batched_transposed_relu_sub(dtype: str = "f32", name: str = "batched_transposed_relu_sub") -> KernelSpec:
    """out[b, n, m] = max(a[b, m, n], 0) - bias[m]: a batch of transposed reads with a row-vector operand.
    Arguments: a [B, M, N], bias [M] -> out [B, N, M]."""
    dims = [("dim_arg0_0", "B"), ("dim_arg0_1", "M"), ("dim_arg0_2", "N")]
    dom = ["dim_arg0_0", "dim_arg0_2", "dim_arg0_1"]
    body = {"domain": dom,
            "loads": [{"arg": 0, "shape": ["dim_arg0_0", "dim_arg0_1", "dim_arg0_2"], "map": [0, 2, 1]},
                      {"arg": 1, "shape": ["dim_arg0_1"], "map": [2]}],
            "store": {"arg": 2, "shape": dom, "map": [0, 1, 2]},
            "body": [op("maximumf", "v0", 0.0), op("subf", "%0", "v1")]}
    return _spec(name, "elementwise", dtype, 2, 1, _EW_TILE, dims, body, _EW_LAUNCH)


def transpose_2d(dtype: str = "f16", name: str = "transpose_2d") -> KernelSpec:
    """out[c, r] = in[r, c]."""
    dims = [("dim_arg0_0", "R"), ("dim_arg0_1", "C")]
    body = {"domain": ["dim_arg0_1", "dim_arg0_0"],
            "loads": [{"arg": 0, "shape": ["dim_arg0_0", "dim_arg0_1"], "map": [1, 0]}],
            "store": {"arg": 1, "shape": ["dim_arg0_1", "dim_arg0_0"], "map": [0, 1]}, "body": []}
    tile = [("WARP_ROWS", 0, (0, 1, 2, 4, 8)), ("CTAS_PER_SM", 0, (0, 4, 8, 16)), ("TILE_KERNEL", 0, (0, 1)),
            ("TILE_ORDER", 0, (0, 1, 2)), ("VARIANT", 0, (0, 1, 2, 3, 4))]
    return _spec(name, "transpose", dtype, 1, 1, tile, dims, body,
                 {"warp_rows": "WARP_ROWS", "ctas_per_sm": "CTAS_PER_SM", "tile_kernel": "TILE_KERNEL",
                  "tile_order": "TILE_ORDER", "variant": "VARIANT"})


# ---- broadcast + add + row reduction -----------------------------------------------------------------
def bcast_add_rowsum(dtype: str = "f32", name: str = "broadcast_add_reducesum") -> KernelSpec:
    """out[m] = sum_n (a[m] + b[m,n]) with f32 accumulation."""
    tile = [("CTA_THREADS", 0, (0, 128, 256, 512)), ("TEAM_LANES", 0, (0, 32, 64, 128, 256)), ("SPLIT_N", 0, (0,)),
            ("BULK_COPY", 1, (1, 0)), ("STREAM_STAGES", 0, (0, 4, 6, 8)), ("STREAM_CHUNK", 0, (0, 2048, 4096, 8192))]
    dims = [("dim_arg0_0", "M"), ("dim_arg1_1", "N")]
    dom = ["dim_arg0_0", "dim_arg1_1"]
    body = {"domain": dom,
            "loads": [{"arg": 0, "shape": ["dim_arg0_0"], "map": [0]}, {"arg": 1, "shape": dom, "map": [0, 1]}],
            "store": {"arg": 2, "shape": ["dim_arg0_0"], "map": [0]},
            "body": [op("addf", "v0", "v1")]}
    return _spec(name, "row_reduce", dtype, 2, 1, tile, dims, body, {"cta_threads": "CTA_THREADS", "team_lanes": "TEAM_LANES", "split_cols": "SPLIT_N", "bulk_copy": "BULK_COPY", "stream_stages": "STREAM_STAGES",
                  "stream_chunk_bytes": "STREAM_CHUNK"})


# ---- gather + elementwise --------------------------------------------------------------------------------
def gather_rows_scale_resid(dtype: str = "bf16", index_dtype: str = "i32", name: str = "gather_scale_resid") -> KernelSpec:
    """out[i,:] = table[idx[i],:] * scale + resid[i,:]."""
    dims = [("dim_arg0_0", "T"), ("dim_arg0_1", "W"), ("dim_arg1_0", "R")]
    dom = ["dim_arg1_0", "dim_arg0_1"]
    body = {"domain": dom,
            "loads": [{"arg": 0, "shape": ["dim_arg0_0", "dim_arg0_1"]},
                      {"arg": 2, "shape": ["dim_arg0_1"], "map": [1]},
                      {"arg": 3, "shape": dom, "map": [0, 1]}],
            "gather": {"axis": 0, "indices": {"arg": 1, "dtype": index_dtype, "shape": ["dim_arg1_0"]}},
            "store": {"arg": 4, "shape": dom, "map": [0, 1]},
            "body": [op("mulf", "v0", "v1"), op("addf", "%0", "v2")]}
    return _spec(name, "gather", dtype, 4, 1, _GATHER_TILE, dims, body, _GATHER_LAUNCH)


def relu_gather_cols_bias(dtype: str = "f16", index_dtype: str = "i64", name: str = "relu_index_select_add") -> KernelSpec:
    """The reference example: out[i,j] = relu(data[i, idx[j]]) + bias[j]."""
    dims = [("dim_arg0_0", "M"), ("dim_arg0_1", "N"), ("dim_arg1_0", "K")]
    dom = ["dim_arg0_0", "dim_arg1_0"]
    body = {"domain": dom,
            "loads": [{"arg": 0, "shape": ["dim_arg0_0", "dim_arg0_1"]}, {"arg": 2, "shape": ["dim_arg1_0"], "map": [1]}],
            "gather": {"axis": 1, "indices": {"arg": 1, "dtype": index_dtype, "shape": ["dim_arg1_0"]}},
            "store": {"arg": 3, "shape": dom, "map": [0, 1]},
            "body": [op("maximumf", "v0", 0.0), op("addf", "%0", "v1")]}
    return _spec(name, "gather", dtype, 3, 1, _GATHER_TILE, dims, body, _GATHER_LAUNCH)


# ---- matmul + bias + LeakyReLU -----------------------------------------------------------------------------
def matmul_bias_leakyrelu(in_dtype: str = "bf16", out_dtype: str = "bf16", bias_dtype: str = "bf16", alpha: float = 0.01,
                          epilogue: str = "BiasAddLeakyRelu", name: str = "matmul_add_leakyrelu",
                          transpose_b: bool = False) -> KernelSpec:
    """E = max(x, alpha*x), x = A[M,K].B[K,N] + bias[N].  Arguments (a, b, bias, out): `out` is the
    reference's init/result tensor (its initial contents are not read).  transpose_b: B is given as [N,K]
    (x = A.B^T, a torch Linear weight); the reference's ABI names the attribute (abi_matmul_trans_b) and always
    sets it false."""
    tile = [("STAGES", 0, (0,))]
    dims = [("dim_arg3_0", "M"), ("dim_arg3_1", "N"), ("dim_arg0_1", "K")]
    body = {"matmul": {"a": 0, "b": 1, "bias": 2, "out": 3, "in_dtype": in_dtype, "out_dtype": out_dtype,
                       "bias_dtype": bias_dtype, "epilogue": epilogue, "alpha": alpha,
                       "m": "dim_arg3_0", "n": "dim_arg3_1", "k": "dim_arg0_1"}}
    if transpose_b:
        body["matmul"]["transpose_b"] = True
    return _spec(name, "matmul", in_dtype, 3, 1, tile, dims, body, {"stages": "STAGES"})
