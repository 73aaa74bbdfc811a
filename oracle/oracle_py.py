"""ctypes/numpy front end to the CPU oracle (``liboracle.so``) and, when it was
built, to the checker library compiled from the reference project's own sources
(``_ref/libkernelh_ref.so``).

TEST INFRASTRUCTURE ONLY. The test suite, the smoke check and the benchmark's
CPU-baseline leg import this module; the product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libkernelh_ref.so")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
_i64 = C.c_int64


def build(force: bool = False) -> None:
    """Compile ``liboracle.so`` (and ``_ref`` when the reference tree exists)."""
    if force or not os.path.exists(_LIB_PATH):
        subprocess.run(["make", "-C", _HERE, "--no-print-directory"], check=True,
                       stdout=subprocess.DEVNULL)


class _CompareResult(C.Structure):
    _fields_ = [("max_abs", C.c_double), ("max_rel_floored", C.c_double), ("max_rel", C.c_double),
                ("rel_frobenius", C.c_double), ("max_violation", C.c_double),
                ("ref_rms", C.c_double), ("non_finite", C.c_int64)]


@dataclass
class Compare:
    max_abs: float
    max_rel_floored: float
    max_rel: float
    rel_frobenius: float
    max_violation: float
    ref_rms: float
    non_finite: int


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.kho_num_threads.restype = C.c_int
        L.kho_set_num_threads.argtypes = [C.c_int]
        L.kho_fill_vecadd_pattern.argtypes = [_f32p, _f32p, _i64]
        L.kho_fill_gemm_pattern.argtypes = [_f32p, _f32p, _i64, _i64, _i64]
        L.kho_fill_lcg.argtypes = [_f32p, _i64, C.POINTER(C.c_uint32)]
        L.kho_fill_mt19937_unit.argtypes = [_f32p, _i64, C.c_uint32]
        L.kho_fill_uniform.argtypes = [_f32p, _i64, C.c_uint64, C.c_double, C.c_double]
        L.kho_fill_normal.argtypes = [_f32p, _i64, C.c_uint64, C.c_double, C.c_double]
        L.kho_vecadd_ref.argtypes = [_f32p, _f32p, _f32p, _i64, C.c_int]
        L.kho_gemm_ref_rows.argtypes = [_f32p, _f32p, _f32p, _i64, _i64, _i64, _i64, _i64, C.c_int]
        L.kho_gemm_ref_pick_rows.argtypes = [_f32p, _f32p, _f32p, _i64, _i64, _i64p, _i64]
        L.kho_softmax_ref.argtypes = [_f32p, _f64p, _i64, _i64, C.c_int]
        L.kho_layernorm_ref.argtypes = [_f32p, _f32p, _f32p, _f64p, _i64, _i64, C.c_double]
        L.kho_scan_ref.argtypes = [_f32p, _f32p, _i64, C.c_int]
        L.kho_fused_gelu_ref.argtypes = [_f32p, _f64p, _i64, C.c_double, C.c_double, C.c_int]
        L.kho_bias_gelu_ref.argtypes = [_f32p, _f32p, _f64p, _i64]
        L.kho_attention_ref.argtypes = [_f32p, _f32p, _f32p, _f64p, _i64, _i64, _i64, _i64,
                                        C.c_int, _i64, _i64]
        L.kho_compare_f32_f64.argtypes = [_f32p, _f64p, _i64, C.c_double, C.POINTER(_CompareResult)]
        L.kho_compare_f32_f32.argtypes = [_f32p, _f32p, _i64, C.c_double, C.POINTER(_CompareResult)]
        L.kho_count_bit_mismatch.argtypes = [_f32p, _f32p, _i64]
        L.kho_count_bit_mismatch.restype = C.c_int64
        L.kho_fnv1a.argtypes = [C.c_void_p, _i64]
        L.kho_fnv1a.restype = C.c_uint64
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().kho_num_threads())


def set_num_threads(n: int) -> None:
    lib().kho_set_num_threads(int(n))


# --------------------------------------------------------------------------- generators
BASE_SEED = 0x4B310001  # synthetic tensors use BASE_SEED + tensor index


def vecadd_pattern(n):
    a = np.empty(n, np.float32)
    b = np.empty(n, np.float32)
    lib().kho_fill_vecadd_pattern(a, b, n)
    return a, b


def gemm_pattern(m, n, k):
    a = np.empty((m, k), np.float32)
    b = np.empty((k, n), np.float32)
    lib().kho_fill_gemm_pattern(a, b, m, n, k)
    return a, b


class LcgStream:
    """The reference tests' 32-bit LCG; one stream may feed several tensors."""

    def __init__(self, seed: int):
        self.seed = C.c_uint32(seed)

    def fill(self, shape) -> np.ndarray:
        v = np.empty(shape, np.float32)
        lib().kho_fill_lcg(v.reshape(-1), v.size, C.byref(self.seed))
        return v


def lcg(shape, seed: int) -> np.ndarray:
    return LcgStream(seed).fill(shape)


def mt19937_unit(n, seed: int) -> np.ndarray:
    v = np.empty(n, np.float32)
    lib().kho_fill_mt19937_unit(v, n, seed)
    return v


def uniform(shape, seed: int, lo: float, hi: float) -> np.ndarray:
    v = np.empty(shape, np.float32)
    lib().kho_fill_uniform(v.reshape(-1), v.size, seed, lo, hi)
    return v


def normal(shape, seed: int, mean: float = 0.0, sigma: float = 1.0) -> np.ndarray:
    v = np.empty(shape, np.float32)
    lib().kho_fill_normal(v.reshape(-1), v.size, seed, mean, sigma)
    return v


# --------------------------------------------------------------------------- references
def vecadd_ref(a, b, subtract=False):
    out = np.empty_like(a)
    lib().kho_vecadd_ref(a, b, out, a.size, int(subtract))
    return out


def gemm_ref(a, b, row_begin=0, row_end=None, b_transposed=False):
    m, k = a.shape
    n = b.shape[0] if b_transposed else b.shape[1]
    row_end = m if row_end is None else row_end
    out = np.empty((row_end - row_begin, n), np.float32)
    lib().kho_gemm_ref_rows(a, b, out, m, n, k, row_begin, row_end, int(b_transposed))
    return out


def gemm_ref_pick_rows(a, b, rows):
    rows = np.ascontiguousarray(rows, np.int64)
    k = a.shape[1]
    n = b.shape[1]
    out = np.empty((rows.size, n), np.float32)
    lib().kho_gemm_ref_pick_rows(a, b, out, n, k, rows, rows.size)
    return out


def softmax_ref(x, uniform_control=False):
    rows, cols = x.shape
    out = np.empty((rows, cols), np.float64)
    lib().kho_softmax_ref(x, out, rows, cols, int(uniform_control))
    return out


def layernorm_ref(x, gamma, beta, eps=1e-5):
    rows, cols = x.shape
    out = np.empty((rows, cols), np.float64)
    lib().kho_layernorm_ref(x, gamma, beta, out, rows, cols, eps)
    return out


def scan_ref(x, exclusive=False):
    out = np.empty_like(x)
    lib().kho_scan_ref(x, out, x.size, int(exclusive))
    return out


def fused_gelu_ref(x, alpha=1.5, beta=0.5, no_tanh_control=False):
    out = np.empty(x.shape, np.float64)
    lib().kho_fused_gelu_ref(x.reshape(-1), out.reshape(-1), x.size, alpha, beta,
                             int(no_tanh_control))
    return out


def bias_gelu_ref(x, bias):
    out = np.empty(x.shape, np.float64)
    lib().kho_bias_gelu_ref(x.reshape(-1), bias.reshape(-1), out.reshape(-1), x.size)
    return out


def attention_ref(q, k, v, scaled=True, bh_begin=0, bh_end=None):
    batch, heads, seq, hd = q.shape
    bh_end = batch * heads if bh_end is None else bh_end
    out = np.zeros(q.shape, np.float64)
    lib().kho_attention_ref(q, k, v, out, batch, heads, seq, hd, int(scaled), bh_begin, bh_end)
    return out


# --------------------------------------------------------------------------- metrics
def compare(got: np.ndarray, ref: np.ndarray, rtol: float = 0.0) -> Compare:
    got = np.ascontiguousarray(got, np.float32).reshape(-1)
    r = _CompareResult()
    if ref.dtype == np.float64:
        lib().kho_compare_f32_f64(got, np.ascontiguousarray(ref).reshape(-1), got.size, rtol,
                                  C.byref(r))
    else:
        lib().kho_compare_f32_f32(got, np.ascontiguousarray(ref, np.float32).reshape(-1),
                                  got.size, rtol, C.byref(r))
    return Compare(r.max_abs, r.max_rel_floored, r.max_rel, r.rel_frobenius, r.max_violation, r.ref_rms,
                   int(r.non_finite))


def bit_mismatches(got: np.ndarray, ref: np.ndarray) -> int:
    return int(lib().kho_count_bit_mismatch(np.ascontiguousarray(got, np.float32).reshape(-1),
                                            np.ascontiguousarray(ref, np.float32).reshape(-1),
                                            got.size))


def fnv1a(arr: np.ndarray) -> int:
    arr = np.ascontiguousarray(arr)
    return int(lib().kho_fnv1a(arr.ctypes.data, arr.nbytes))


# --------------------------------------------------------------------------- the reference's own code
def ref_available() -> bool:
    return os.path.exists(_REF_PATH)


_ref = None


def ref():
    """The library compiled from the reference project's own sources."""
    global _ref
    if _ref is None:
        R = C.CDLL(_REF_PATH)
        u32p = C.POINTER(C.c_uint)
        R.khref_softmax_fill.argtypes = [_f32p, C.c_long, u32p]
        R.khref_softmax_ref.argtypes = [_f32p, _f64p, C.c_long, C.c_long]
        R.khref_layernorm_fill.argtypes = [_f32p, C.c_long, u32p]
        R.khref_layernorm_ref.argtypes = [_f32p, _f32p, _f32p, _f64p, C.c_long, C.c_long,
                                          C.c_double]
        R.khref_gelu_fill.argtypes = [_f32p, C.c_long, u32p]
        R.khref_gelu_ref.argtypes = [_f32p, _f64p, C.c_long, C.c_int]
        R.khref_attention_fill.argtypes = [_f32p, C.c_long, C.c_uint]
        R.khref_attention_ref.argtypes = [_f32p, _f32p, _f32p, _f64p, C.c_long, C.c_long, C.c_int]
        R.khref_gemm_fill.argtypes = [_f32p, _f32p, C.c_long, C.c_long, C.c_long]
        R.khref_gemm_ref.argtypes = [_f32p, _f32p, _f32p, C.c_long, C.c_long, C.c_long]
        R.khref_gemm_rel_frobenius.argtypes = [_f32p, _f32p, C.c_long]
        R.khref_gemm_rel_frobenius.restype = C.c_double
        R.khref_gemm_prepare.argtypes = [_f32p, C.c_long, C.c_long]
        R.khref_gemm_prepare.restype = C.c_void_p
        R.khref_gemm_rows.argtypes = [C.c_void_p, _f32p, _f32p, C.c_long]
        R.khref_gemm_release.argtypes = [C.c_void_p]
        R.khref_vecadd_fill.argtypes = [_f32p, _f32p, C.c_long]
        R.khref_scan_fill.argtypes = [_f32p, C.c_long, C.c_uint]
        R.khref_pack_memrefs.argtypes = [C.POINTER(C.c_ulonglong), C.POINTER(C.c_longlong),
                                         C.POINTER(C.c_int), C.c_int,
                                         C.POINTER(C.c_ulonglong), C.c_int]
        R.khref_device_limits.argtypes = [C.c_char_p, C.POINTER(C.c_longlong), C.c_char_p,
                                          C.c_int, C.c_char_p, C.c_int]
        R.khref_verify_launch.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_ulonglong, C.c_int, C.c_char_p, C.c_int]
        R.khref_occupancy.argtypes = [C.c_char_p, C.c_int, C.c_long, C.c_int, C.POINTER(C.c_int)]
        R.khref_occupancy.restype = C.c_double
        R.khref_metric.argtypes = [C.c_char_p, C.c_long, C.c_long, C.c_long, C.c_long]
        R.khref_metric.restype = C.c_double
        R.khref_rate.argtypes = [C.c_int, C.c_double, C.c_double]
        R.khref_rate.restype = C.c_double
        R.khref_csv_line.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_double, C.c_double,
                                     C.c_char_p, C.c_char_p, C.c_char_p, C.c_int]
        R.khref_csv_header.argtypes = [C.c_char_p, C.c_int]
        R.khref_shape_roundtrip.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        _ref = R
    return _ref
