"""ctypes binding of liboracle_cpu.so (oracle_cpu.c).  TEST INFRASTRUCTURE ONLY: used by the
tests, the smoke entry and the benchmark's CPU-baseline / reference legs as the checker or the
timed CPU baseline - never by the shipped package."""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_double, c_float, c_int, c_int64, c_longlong, c_uint8, c_uint16, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle_cpu.so")
_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} missing: run `make -C {_HERE}`")
        lib = ctypes.CDLL(LIB_PATH)
        lib.oracle_num_threads.restype = c_int
        lib.oracle_set_num_threads.argtypes = [c_int]
        lib.oracle_dequant_bf16.argtypes = [c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.oracle_skinny_gemm.argtypes = [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                           c_void_p, c_void_p]
        lib.oracle_chain_f32.argtypes = [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]
        lib.oracle_argmax_rows.argtypes = [c_int, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p]
        _lib = lib
    return _lib


def _ptr(a):
    return a.ctypes.data_as(c_void_p) if a is not None else None


def num_threads() -> int:
    return load().oracle_num_threads()


def set_num_threads(n: int) -> None:
    """Threads of the OpenMP loops from here on (overrides OMP_NUM_THREADS)."""
    load().oracle_set_num_threads(int(max(1, n)))


def dequant_bf16(mode, w, n_cols, col_offset=0, w_scale=None):
    w = np.ascontiguousarray(w)
    K = w.shape[0]
    row_stride = w.shape[1] if mode != 2 else w.shape[1] * 16 // 9
    s = None if w_scale is None else np.ascontiguousarray(w_scale, dtype=np.float32)
    out = np.empty((K, n_cols), dtype=np.uint16)
    load().oracle_dequant_bf16(mode, _ptr(w.view(np.uint8)), K, row_stride, col_offset, n_cols, _ptr(s), _ptr(out))
    return out


def skinny_gemm(mode, x_bits, w, n, w_scale=None, want_sums=True):
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w = np.ascontiguousarray(w)
    M, K = x.shape
    s = None if w_scale is None else np.ascontiguousarray(w_scale, dtype=np.float32)
    out = np.empty((M, n), dtype=np.uint16)
    sums = np.empty((M, n), dtype=np.float64) if want_sums else None
    mags = np.empty((M, n), dtype=np.float64) if want_sums else None
    load().oracle_skinny_gemm(mode, _ptr(x), M, K, _ptr(w.view(np.uint8)), n, _ptr(s), _ptr(out), _ptr(sums),
                              _ptr(mags))
    return out, sums, mags


def chain_f32(mode, x_bits, w, n, w_scale=None):
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w = np.ascontiguousarray(w)
    M, K = x.shape
    s = None if w_scale is None else np.ascontiguousarray(w_scale, dtype=np.float32)
    out = np.empty((M, n), dtype=np.uint16)
    load().oracle_chain_f32(mode, _ptr(x), M, K, _ptr(w.view(np.uint8)), n, _ptr(s), _ptr(out))
    return out


def argmax_rows(dtype_code, x):
    """dtype_code: 0 BF16 bits (uint16), 1 FP16 bits (uint16), 2 float32."""
    x = np.ascontiguousarray(x)
    rows, V = x.shape
    idx = np.empty(rows, dtype=np.int64)
    val = np.empty(rows, dtype=np.float32)
    load().oracle_argmax_rows(dtype_code, _ptr(x), rows, V, _ptr(idx), _ptr(val))
    return idx, val
