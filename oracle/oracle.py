"""ctypes front for the CPU oracle (libafir_oracle.so, built by oracle/Makefile).

TEST INFRASTRUCTURE ONLY.  Importable from tests/, the smoke check and the
bench's CPU-baseline leg; the shipped package never imports this module.
16-bit float tensors travel as numpy uint16 bit patterns (float16 arrays are
viewed, bf16 has no numpy dtype).
"""
import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None

_i64 = ctypes.c_int64
_p = ctypes.c_void_p


def build(force: bool = False) -> Path:
    so = _HERE / "libafir_oracle.so"
    src = _HERE / "afir_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, stdout=subprocess.DEVNULL)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(str(build()))
        _LIB.afo_num_threads.restype = ctypes.c_int
        _LIB.afo_gather_rows_scale_resid_bf16.restype = _i64
        _LIB.afo_relu_gather_cols_bias_f16.restype = _i64
        _LIB.afo_compare_f32.restype = _i64
        _LIB.afo_matmul_bias_leakyrelu_bf16_at.restype = ctypes.c_double
    return _LIB


def num_threads() -> int:
    return int(lib().afo_num_threads())


def set_num_threads(n: int) -> None:
    lib().afo_set_num_threads(ctypes.c_int(n))


def _ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle wants C-contiguous arrays"
    return _p(a.ctypes.data)


def _u16(a: np.ndarray) -> np.ndarray:
    """float16 -> uint16 view; uint16 passes through."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        return a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return a


# ---- conversions -----------------------------------------------------------
def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().afo_f32_to_bf16(_ptr(x), _ptr(out), _i64(x.size))
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().afo_bf16_to_f32(_ptr(x), _ptr(out), _i64(x.size))
    return out


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().afo_f32_to_f16(_ptr(x), _ptr(out), _i64(x.size))
    return out


def f16_bits_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().afo_f16_to_f32(_ptr(x), _ptr(out), _i64(x.size))
    return out


# ---- elementwise chains ----------------------------------------------------
def add_mul_f32(a, b):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    out = np.empty_like(a)
    lib().afo_add_mul_f32(_ptr(a), _ptr(b), _ptr(out), _i64(a.size))
    return out


def split_relu_bias_mul_f16(x, bias, bias_axis=1):
    x, bias = _u16(x), _u16(bias)
    B, R, C2 = x.shape
    C = C2 // 2
    out = np.empty((B, R, C), np.uint16)
    lib().afo_split_relu_bias_mul_f16(_ptr(x), _ptr(bias), _ptr(out), _i64(B), _i64(R), _i64(C),
                                      ctypes.c_int(bias_axis))
    return out.view(np.float16)


def split_rows_relu_bias_scale_f16(a, bias0, bias1, scale0, scale1):
    a, bias0, bias1, scale0, scale1 = map(_u16, (a, bias0, bias1, scale0, scale1))
    M, N = a.shape
    out = np.empty((M, N), np.uint16)
    lib().afo_split_rows_relu_bias_scale_f16(_ptr(a), _ptr(bias0), _ptr(bias1), _ptr(scale0), _ptr(scale1),
                                             _ptr(out), _i64(M), _i64(N))
    return out.view(np.float16)


def add_mul_concat_f16(a, b, c, d):
    a, b, c, d = map(_u16, (a, b, c, d))
    M, N = b.shape
    out = np.empty((2 * M, N), np.uint16)
    lib().afo_add_mul_concat_f16(_ptr(a), _ptr(b), _ptr(c), _ptr(d), _ptr(out), _i64(M), _i64(N))
    return out.view(np.float16)


def relu_bcast_transpose_add_f16(d0, d1):
    d0, d1 = _u16(d0), _u16(d1)
    N, M = d1.shape
    out = np.empty((N, M), np.uint16)
    lib().afo_relu_bcast_transpose_add_f16(_ptr(d0), _ptr(d1), _ptr(out), _i64(M), _i64(N))
    return out.view(np.float16)


def transpose_2d(x):
    x = np.ascontiguousarray(x)
    M, N = x.shape
    out = np.empty((N, M), x.dtype)
    lib().afo_transpose_2d(_ptr(x), _ptr(out), _i64(M), _i64(N), ctypes.c_int(x.dtype.itemsize))
    return out


# ---- reductions ------------------------------------------------------------
def bcast_add_rowsum_f32(a, b, with_bounds=False):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    M, N = b.shape
    out = np.empty(M, np.float32)
    if not with_bounds:
        lib().afo_bcast_add_rowsum_f32_fast(_ptr(a), _ptr(b), _ptr(out), _i64(M), _i64(N))
        return out
    s64 = np.empty(M, np.float64)
    a64 = np.empty(M, np.float64)
    lib().afo_bcast_add_rowsum_f32(_ptr(a), _ptr(b), _ptr(out), _ptr(s64), _ptr(a64), _i64(M), _i64(N))
    return out, s64, a64


def bcast_add_rowsum_f16(a, b):
    a, b = _u16(a), _u16(b)
    M, N = b.shape
    out = np.empty(M, np.uint16)
    lib().afo_bcast_add_rowsum_f16(_ptr(a), _ptr(b), _ptr(out), _i64(M), _i64(N))
    return out.view(np.float16)


# ---- gather ----------------------------------------------------------------
def gather_rows_scale_resid_bf16(table, idx, scale, resid):
    table, scale, resid = (np.ascontiguousarray(t, np.uint16) for t in (table, scale, resid))
    idx = np.ascontiguousarray(idx, np.int32)
    rows, width = resid.shape
    out = np.zeros((rows, width), np.uint16)
    bad = lib().afo_gather_rows_scale_resid_bf16(_ptr(table), _ptr(idx), _ptr(scale), _ptr(resid), _ptr(out),
                                                 _i64(rows), _i64(width), _i64(table.shape[0]))
    if bad:
        raise IndexError(f"{bad} gather indices out of range")
    return out


def relu_gather_cols_bias_f16(data, idx, bias):
    data, bias = _u16(data), _u16(bias)
    idx = np.ascontiguousarray(idx, np.int64)
    M, N = data.shape
    K = idx.shape[0]
    out = np.empty((M, K), np.uint16)
    bad = lib().afo_relu_gather_cols_bias_f16(_ptr(data), _ptr(idx), _ptr(bias), _ptr(out), _i64(M), _i64(N),
                                              _i64(K))
    if bad:
        raise IndexError(f"{bad} gather indices out of range")
    return out.view(np.float16)


# ---- matmul ----------------------------------------------------------------
def matmul_bias_leakyrelu_bf16(A, B, bias, alpha, row_begin=0, row_end=None):
    A, B, bias = (np.ascontiguousarray(t, np.uint16) for t in (A, B, bias))
    M, K = A.shape
    N = B.shape[1]
    row_end = M if row_end is None else row_end
    out = np.zeros((M, N), np.uint16)
    lib().afo_matmul_bias_leakyrelu_bf16(_ptr(A), _ptr(B), _ptr(bias), _ptr(out), _i64(M), _i64(N), _i64(K),
                                         ctypes.c_float(alpha), _i64(row_begin), _i64(row_end))
    return out


def matmul_bias_leakyrelu_f16_f32(A, B, bias, alpha):
    A, B = _u16(A), _u16(B)
    bias = np.ascontiguousarray(bias, np.float32)
    M, K = A.shape
    N = B.shape[1]
    out = np.zeros((M, N), np.float32)
    lib().afo_matmul_bias_leakyrelu_f16_f32(_ptr(A), _ptr(B), _ptr(bias), _ptr(out), _i64(M), _i64(N), _i64(K),
                                            ctypes.c_float(alpha), _i64(0), _i64(M))
    return out


def matmul_bias_leakyrelu_bf16_at(A, B, bias, alpha, m, n):
    A, B, bias = (np.ascontiguousarray(t, np.uint16) for t in (A, B, bias))
    K = A.shape[1]
    N = B.shape[1]
    return float(lib().afo_matmul_bias_leakyrelu_bf16_at(_ptr(A), _ptr(B), _ptr(bias), _i64(N), _i64(K),
                                                         ctypes.c_float(alpha), _i64(m), _i64(n)))


# ---- comparator ------------------------------------------------------------
def compare(actual, expected, atol, rtol):
    """Reference comparator rule; returns (fails, max_abs, mean_abs)."""
    a = np.ascontiguousarray(actual, np.float32).ravel()
    e = np.ascontiguousarray(expected, np.float32).ravel()
    assert a.size == e.size
    mx, mean = ctypes.c_double(), ctypes.c_double()
    fails = lib().afo_compare_f32(_ptr(a), _ptr(e), _i64(a.size), ctypes.c_double(atol), ctypes.c_double(rtol),
                                  ctypes.byref(mx), ctypes.byref(mean))
    return int(fails), mx.value, mean.value
