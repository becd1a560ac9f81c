"""ctypes binding of libqfg_b200.so (the C ABI declared in include/qfg.h).

The shared library is built in-tree by `make -C qwen38_flash_ops_b200/csrc` (or
`__graft_entry__.build()`).  There is no fallback: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
# QFG_LIBRARY names another build of the same library (a measurement build, for instance)
LIB_PATH = os.environ.get("QFG_LIBRARY") or os.path.join(_HERE, "libqfg_b200.so")

QFG_OK, QFG_FAIL, QFG_INVALID_ARGUMENT = 0, 1, 2
QFG_FLOAT, QFG_UINT8, QFG_INT64, QFG_FLOAT16, QFG_BFLOAT16, QFG_FLOAT8E4M3FN = 1, 2, 7, 10, 16, 17

# every symbol include/qfg.h declares
EXPORTS = (
    "qfg_last_error", "qfg_version",
    "qfg_skinny_gemm_create", "qfg_skinny_gemm_compute", "qfg_skinny_gemm_set_option",
    "qfg_skinny_gemm_describe", "qfg_plan_describe", "qfg_skinny_gemm_destroy",
    "qfg_argmax_rows",
    "qfg_dequant_create", "qfg_dequant_compute", "qfg_dequant_destroy",
    "qfg_untile_hc_create", "qfg_untile_hc_compute", "qfg_untile_hc_destroy",
    "qfg_shared_expert_down_create", "qfg_shared_expert_down_compute", "qfg_shared_expert_down_set_option",
    "qfg_shared_expert_down_destroy",
    "qfg_lmhead_workspace_bytes", "qfg_lmhead_create", "qfg_lmhead_compute", "qfg_lmhead_static_max_rows",
    "qfg_lmhead_compute_static", "qfg_lmhead_set_option",
    "qfg_lmhead_destroy", "qfg_lmhead_combine",
    "qfg_lmhead_exchange_bytes", "qfg_lmhead_compute_sharded", "qfg_lmhead_exchange_status",
    "qfg_lmhead_exchange_times",
    "qfg_peer_alloc", "qfg_peer_open", "qfg_peer_close", "qfg_peer_free",
    "qfg_lmhead_host_create", "qfg_lmhead_host_run", "qfg_lmhead_host_destroy",
    "qfg_stream_read_probe",
)


class LmExchange(ctypes.Structure):
    _fields_ = [("world", c_int), ("rank", c_int), ("peers", c_void_p * 8)]


class Tensor2D(ctypes.Structure):
    _fields_ = [("data", c_void_p), ("dtype", c_int32), ("rows", c_int64), ("cols", c_int64)]


class QfgError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}`; "
            "this package has no fallback implementation")
    lib = ctypes.CDLL(LIB_PATH)
    lib.qfg_last_error.restype = c_char_p
    lib.qfg_version.restype = c_char_p
    lib.qfg_skinny_gemm_create.argtypes = [POINTER(c_int64), c_int, POINTER(c_int64), c_int, POINTER(c_float),
                                           c_size_t, c_int, POINTER(c_void_p)]
    lib.qfg_skinny_gemm_compute.argtypes = [c_void_p, c_void_p, c_int64, c_int64, POINTER(Tensor2D), c_int,
                                            POINTER(c_void_p), c_int, c_void_p]
    lib.qfg_skinny_gemm_set_option.argtypes = [c_void_p, c_char_p, c_char_p]
    lib.qfg_skinny_gemm_describe.argtypes = [c_void_p, c_int64, POINTER(Tensor2D), c_int, c_char_p, c_size_t]
    lib.qfg_plan_describe.argtypes = [c_int, c_int64, POINTER(c_int64), c_int, c_int, c_int, c_char_p, c_char_p,
                                      c_size_t]
    lib.qfg_skinny_gemm_destroy.argtypes = [c_void_p]
    lib.qfg_skinny_gemm_destroy.restype = None
    lib.qfg_argmax_rows.argtypes = [c_int, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]
    lib.qfg_dequant_create.argtypes = [c_int64, c_int64, POINTER(c_int64), c_int, POINTER(c_float), c_size_t,
                                       POINTER(c_void_p)]
    lib.qfg_dequant_compute.argtypes = [c_void_p, POINTER(Tensor2D), POINTER(c_void_p), c_int, c_void_p]
    lib.qfg_dequant_destroy.argtypes = [c_void_p]
    lib.qfg_dequant_destroy.restype = None
    lib.qfg_lmhead_workspace_bytes.restype = c_size_t
    lib.qfg_lmhead_create.argtypes = [POINTER(c_float), c_size_t, c_int, POINTER(c_void_p)]
    lib.qfg_lmhead_compute.argtypes = [c_void_p, c_void_p, c_int64, c_int64, POINTER(Tensor2D), c_int64, c_int64,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.qfg_lmhead_static_max_rows.restype = c_size_t
    lib.qfg_lmhead_compute_static.argtypes = [c_void_p, c_void_p, c_int64, c_int64, POINTER(Tensor2D), c_int64, c_int64,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.qfg_shared_expert_down_create.argtypes = [POINTER(c_float), c_size_t, c_int, POINTER(c_void_p)]
    lib.qfg_shared_expert_down_compute.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, POINTER(Tensor2D), c_void_p,
                                                   c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]
    lib.qfg_shared_expert_down_set_option.argtypes = [c_void_p, c_char_p, c_char_p]
    lib.qfg_shared_expert_down_destroy.argtypes = [c_void_p]
    lib.qfg_shared_expert_down_destroy.restype = None
    lib.qfg_untile_hc_create.argtypes = [c_int, POINTER(c_float), c_size_t, POINTER(c_void_p)]
    lib.qfg_untile_hc_compute.argtypes = [c_void_p, POINTER(Tensor2D), c_void_p, c_void_p]
    lib.qfg_untile_hc_destroy.argtypes = [c_void_p]
    lib.qfg_untile_hc_destroy.restype = None
    lib.qfg_lmhead_exchange_bytes.restype = c_size_t
    lib.qfg_lmhead_compute_sharded.argtypes = [c_void_p, c_void_p, c_int64, c_int64, POINTER(Tensor2D), c_int64, c_int64,
                                               c_void_p, POINTER(LmExchange), c_void_p, c_void_p, c_void_p, c_void_p]
    lib.qfg_lmhead_exchange_status.argtypes = [c_void_p, POINTER(c_int)]
    lib.qfg_lmhead_exchange_times.argtypes = [c_void_p, POINTER(c_uint64)]
    lib.qfg_lmhead_host_create.argtypes = [c_void_p, c_int64, c_int64, POINTER(Tensor2D), c_int64, c_int64, c_void_p,
                                           POINTER(LmExchange), c_void_p, c_void_p, c_void_p, c_void_p, POINTER(c_void_p)]
    lib.qfg_stream_read_probe.argtypes = [c_void_p, c_size_t, c_void_p, c_void_p]
    lib.qfg_lmhead_host_run.argtypes = [c_void_p]
    lib.qfg_lmhead_host_destroy.argtypes = [c_void_p]
    lib.qfg_lmhead_host_destroy.restype = None
    lib.qfg_peer_alloc.argtypes = [c_size_t, POINTER(c_void_p), ctypes.c_char_p]
    lib.qfg_peer_open.argtypes = [ctypes.c_char_p, POINTER(c_void_p)]
    lib.qfg_peer_close.argtypes = [c_void_p]
    lib.qfg_peer_free.argtypes = [c_void_p]
    lib.qfg_lmhead_set_option.argtypes = [c_void_p, c_char_p, c_char_p]
    lib.qfg_lmhead_destroy.argtypes = [c_void_p]
    lib.qfg_lmhead_destroy.restype = None
    lib.qfg_lmhead_combine.argtypes = [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != QFG_OK:
        raise QfgError(code, load().qfg_last_error().decode())


def plan_describe(dtype: int, k: int, n, row_align: int = 16, sm_count: int = 148, spec: str = "") -> dict:
    """The launch plan for a shape as a dict (needs no GPU)."""
    buf = ctypes.create_string_buffer(512)
    arr = i64_array(n)
    check(load().qfg_plan_describe(dtype, k, arr, len(n), row_align, sm_count, spec.encode(), buf, 512))
    out = {}
    for item in buf.value.decode().split(","):
        key, val = item.split("=")
        out[key] = [int(v) for v in val.split("/")] if key == "seg_tiles" else int(val)
    return out


def i64_array(values):
    arr = (c_int64 * len(values))(*[int(v) for v in values])
    return arr


def f32_array(values):
    import numpy as np

    a = np.ascontiguousarray(values, dtype=np.float32)
    return a, a.ctypes.data_as(POINTER(c_float))
