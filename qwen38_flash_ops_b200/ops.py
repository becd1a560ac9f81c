"""Python mirror of the `qwen.fused_gemm` operators, over the C ABI.

Each class corresponds to one custom op of the reference library and keeps its names,
attributes and argument order (SkinnyGemmOp / ArgmaxRowsOp / DequantWeightBf16Op,
src/fused_gemm/fused_gemm.cu:781-840, :956-977): attributes go to the constructor (kernel
creation in ORT), tensors to `__call__` (ComputeV2), outputs are allocated here the way ORT
allocates them.  torch is used only to hold device memory and streams; all arithmetic runs in
libqfg_b200.so on the current CUDA stream.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p

import torch

from . import _lib
from ._lib import QfgError, Tensor2D, check

_DTYPES = {
    torch.bfloat16: _lib.QFG_BFLOAT16,
    torch.float16: _lib.QFG_FLOAT16,
    torch.float32: _lib.QFG_FLOAT,
    torch.uint8: _lib.QFG_UINT8,
    torch.float8_e4m3fn: _lib.QFG_FLOAT8E4M3FN,
}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _tensor2d(w: torch.Tensor) -> Tensor2D:
    if w.dim() != 2:
        raise QfgError(_lib.QFG_INVALID_ARGUMENT, "weight must be a 2-D tensor")
    if not w.is_cuda or not w.is_contiguous():
        raise QfgError(_lib.QFG_INVALID_ARGUMENT, "weight must be a contiguous CUDA tensor")
    if w.dtype not in _DTYPES:
        raise QfgError(_lib.QFG_INVALID_ARGUMENT, f"unsupported weight element type {w.dtype}")
    return Tensor2D(w.data_ptr(), _DTYPES[w.dtype], w.shape[0], w.shape[1])


def _require_cuda(x: torch.Tensor, what: str) -> None:
    if not x.is_cuda or not x.is_contiguous():
        raise QfgError(_lib.QFG_INVALID_ARGUMENT, f"{what} must be a contiguous CUDA tensor")


class SkinnyGemm:
    """y_j = x[..., K] @ W_i[K, N_i], column-sliced over the outputs listed in `widths`.

    Attributes as in the reference node: `seg_outs` (outputs per weight), `widths`, optional
    `w_scale` (concatenated per-column scales of the quantised weights), optional `trigger`.
    Weights: torch.bfloat16 [K, N], torch.float8_e4m3fn [K, N] or torch.uint8 [K, N*9/16] (NVFP4).
    """

    def __init__(self, seg_outs, widths, w_scale=None, trigger: int = 0):
        lib = _lib.load()
        self._lib = lib
        self._h = c_void_p()
        so, wi = _lib.i64_array(seg_outs), _lib.i64_array(widths)
        if w_scale is not None and len(w_scale) > 0:
            keep, ptr = _lib.f32_array(w_scale)
            n = keep.size
        else:
            keep, ptr, n = None, None, 0
        check(lib.qfg_skinny_gemm_create(so, len(seg_outs), wi, len(widths), ptr, n, int(trigger),
                                         ctypes.byref(self._h)))
        self.seg_outs = [int(v) for v in seg_outs]
        self.widths = [int(v) for v in widths]

    def set_option(self, key: str, value) -> None:
        check(self._lib.qfg_skinny_gemm_set_option(self._h, key.encode(), str(value).encode()))

    def describe(self, k: int, *weights: torch.Tensor) -> str:
        arr = (Tensor2D * len(weights))(*[_tensor2d(w) for w in weights])
        buf = ctypes.create_string_buffer(512)
        check(self._lib.qfg_skinny_gemm_describe(self._h, k, arr, len(weights), buf, 512))
        return buf.value.decode()

    def __call__(self, x: torch.Tensor, *weights: torch.Tensor, out=None):
        _require_cuda(x, "x")
        if x.dtype != torch.bfloat16:
            raise QfgError(_lib.QFG_INVALID_ARGUMENT, "SkinnyGemm: x must be BF16")
        k = x.shape[-1]
        m = x.numel() // k if k > 0 else 0
        lead = tuple(x.shape[:-1])
        if out is None:
            out = [torch.empty(lead + (w,), dtype=torch.bfloat16, device=x.device) for w in self.widths]
        arr = (Tensor2D * max(len(weights), 1))(*[_tensor2d(w) for w in weights])
        outs = (c_void_p * max(len(out), 1))(*[o.data_ptr() for o in out])
        check(self._lib.qfg_skinny_gemm_compute(self._h, x.data_ptr(), m, k, arr, len(weights), outs, len(out),
                                                _stream_ptr()))
        return out

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.qfg_skinny_gemm_destroy(h)
            self._h = None


class ArgmaxRows:
    """idx[...] = argmax over the last axis of BF16 / FP16 / FP32 logits, numpy semantics;
    optionally also the maximum as FP32.  The output rank is the input rank minus one."""

    def __init__(self):
        self._lib = _lib.load()

    def __call__(self, x: torch.Tensor, with_val: bool = True, out=None):
        """`out`: optional (idx, val) tensors to write into (val may be None)."""
        _require_cuda(x, "x")
        if x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise QfgError(_lib.QFG_INVALID_ARGUMENT, "ArgmaxRows: logits must be BF16/FP16/FP32")
        if x.dim() == 0 or x.shape[-1] < 1:
            raise QfgError(_lib.QFG_INVALID_ARGUMENT, "ArgmaxRows: bad shape")
        vocab = x.shape[-1]
        lead = tuple(x.shape[:-1])
        rows = x.numel() // vocab
        if out is not None:
            idx, val = out
            with_val = val is not None
        else:
            idx = torch.empty(lead, dtype=torch.int64, device=x.device)
            val = torch.empty(lead, dtype=torch.float32, device=x.device) if with_val else None
        check(self._lib.qfg_argmax_rows(_DTYPES[x.dtype], x.data_ptr(), rows, vocab, idx.data_ptr(),
                                        val.data_ptr() if with_val else None, _stream_ptr()))
        return (idx, val) if with_val else idx


class DequantWeightBf16:
    """A column slice of a BF16 / FP8 / NVFP4 weight as BF16, split over `widths` outputs.
    Attributes: `n_cols` (required), `col_offset`, `widths`, `w_scale` (per output column).
    The optional second input of the reference op is unused there and omitted here."""

    def __init__(self, n_cols: int, col_offset: int = 0, widths=None, w_scale=None):
        lib = _lib.load()
        self._lib = lib
        self._h = c_void_p()
        widths = list(widths) if widths else []
        wi = _lib.i64_array(widths) if widths else None
        if w_scale is not None and len(w_scale) > 0:
            keep, ptr = _lib.f32_array(w_scale)
            n = keep.size
        else:
            keep, ptr, n = None, None, 0
        check(lib.qfg_dequant_create(int(n_cols), int(col_offset), wi, len(widths), ptr, n, ctypes.byref(self._h)))
        self.widths = widths if widths else [int(n_cols)]

    def __call__(self, w: torch.Tensor, out=None):
        t = _tensor2d(w)
        outs = out if out is not None else [torch.empty((w.shape[0], wd), dtype=torch.bfloat16, device=w.device) for wd in self.widths]
        ptrs = (c_void_p * len(outs))(*[o.data_ptr() for o in outs])
        check(self._lib.qfg_dequant_compute(self._h, ctypes.byref(t), ptrs, len(outs), _stream_ptr()))
        return outs

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.qfg_dequant_destroy(h)
            self._h = None


class SharedExpertDown:
    """y = routed + bf16(bf16(swish_mul(g, u) @ W) * bf16(sigmoid(bf16(dot(gx, gw))))) per row.
    Inputs as the reference node: g, u BF16 [..., K]; W [K, N] (BF16 / FP8) or UINT8 [K, 9N/16] (NVFP4);
    gx BF16 [..., gk]; gw BF16 [gk, 1]; routed BF16 [..., N].  Attributes: optional `w_scale`, `trigger`."""

    def __init__(self, w_scale=None, trigger: int = 0):
        lib = _lib.load()
        self._lib = lib
        self._h = c_void_p()
        if w_scale is not None and len(w_scale) > 0:
            keep, ptr = _lib.f32_array(w_scale)
            n = keep.size
        else:
            keep, ptr, n = None, None, 0
        check(lib.qfg_shared_expert_down_create(ptr, n, int(trigger), ctypes.byref(self._h)))

    def set_option(self, key: str, value) -> None:
        check(self._lib.qfg_shared_expert_down_set_option(self._h, key.encode(), str(value).encode()))

    def __call__(self, g, u, w, gx, gw, routed):
        for name, t in (("g", g), ("u", u), ("gx", gx), ("gw", gw), ("routed", routed)):
            _require_cuda(t, name)
            if t.dtype != torch.bfloat16:
                raise QfgError(_lib.QFG_FAIL, f"SharedExpertDown: {name} must be BF16")
        k = w.shape[0]
        n = routed.shape[-1]
        m = g.numel() // k if k > 0 else 0
        gk = gw.numel()
        if (m < 1 or g.numel() != m * k or u.numel() != m * k or routed.numel() != m * n or gx.numel() != m * gk
                or gw.shape[-1] != 1):
            raise QfgError(_lib.QFG_FAIL, "SharedExpertDown: shape mismatch")
        t = _tensor2d(w)
        if w.dtype == torch.uint8:
            if n % 16 != 0 or w.shape[1] != n * 9 // 16:
                raise QfgError(_lib.QFG_FAIL, "SharedExpertDown: NVFP4 weight N mismatch")
        elif w.shape[1] != n:
            raise QfgError(_lib.QFG_FAIL, "SharedExpertDown: weight N mismatch")
        out = torch.empty_like(routed)
        check(self._lib.qfg_shared_expert_down_compute(self._h, g.data_ptr(), u.data_ptr(), m, k, ctypes.byref(t), gx.data_ptr(),
                                                       gk, gw.data_ptr(), routed.data_ptr(), n, out.data_ptr(), _stream_ptr()))
        return out

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.qfg_shared_expert_down_destroy(h)
            self._h = None


class UntileHcBf16:
    """The pre-tiled hyper-connection weight [160, 20480] (BF16, or FP8 E4M3FN with a per-output-column
    `w_scale`) as row-major BF16: [10240, 320] for kind 0, [320, 10240] for kind 1.  The optional second
    input of the reference op only ties buffer lifetimes and is omitted here."""

    def __init__(self, kind: int, w_scale=None):
        lib = _lib.load()
        self._lib = lib
        self._h = c_void_p()
        self.kind = int(kind)
        if w_scale is not None and len(w_scale) > 0:
            keep, ptr = _lib.f32_array(w_scale)
            n = keep.size
        else:
            keep, ptr, n = None, None, 0
        check(lib.qfg_untile_hc_create(self.kind, ptr, n, ctypes.byref(self._h)))

    def __call__(self, w: torch.Tensor, out=None):
        _require_cuda(w, "w")
        t = _tensor2d(w)
        shape = (10240, 320) if self.kind == 0 else (320, 10240)
        if out is None:
            out = torch.empty(shape, dtype=torch.bfloat16, device=w.device)
        elif tuple(out.shape) != shape or out.dtype != torch.bfloat16 or not out.is_contiguous():
            raise QfgError(_lib.QFG_INVALID_ARGUMENT, "UntileHcBf16: out must be a contiguous BF16 tensor of the untiled shape")
        check(self._lib.qfg_untile_hc_compute(self._h, ctypes.byref(t), out.data_ptr(), _stream_ptr()))
        return out

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.qfg_untile_hc_destroy(h)
            self._h = None


class LmHeadArgmax:
    """SkinnyGemm over one LM-head weight fused with ArgmaxRows over the BF16-rounded logits.

    Returns (idx int64 [m], val float32 [m], key uint64-as-int64 [m]); `key` orders
    (value, index) pairs like ArgmaxRows does and is what the N-sharded head all-gathers.
    The instance owns a zeroed workspace (about 256 KB); calls on one instance must not overlap on the GPU.
    """

    def __init__(self, w_scale=None, trigger: int = 0, device="cuda"):
        lib = _lib.load()
        self._lib = lib
        self._h = c_void_p()
        if w_scale is not None and len(w_scale) > 0:
            keep, ptr = _lib.f32_array(w_scale)
            n = keep.size
        else:
            keep, ptr, n = None, None, 0
        check(lib.qfg_lmhead_create(ptr, n, int(trigger), ctypes.byref(self._h)))
        self.workspace = torch.zeros(lib.qfg_lmhead_workspace_bytes(), dtype=torch.uint8, device=device)

    def set_option(self, key: str, value) -> None:
        check(self._lib.qfg_lmhead_set_option(self._h, key.encode(), str(value).encode()))

    def __call__(self, x: torch.Tensor, w: torch.Tensor, n: int, col_offset: int = 0, logits: bool = False,
                 out=None):
        _require_cuda(x, "x")
        if x.dtype != torch.bfloat16:
            raise QfgError(_lib.QFG_INVALID_ARGUMENT, "LmHead: x must be BF16")
        k = x.shape[-1]
        m = x.numel() // k
        t = _tensor2d(w)
        if out is None:
            idx = torch.empty(m, dtype=torch.int64, device=x.device)
            val = torch.empty(m, dtype=torch.float32, device=x.device)
            key = torch.empty(m, dtype=torch.int64, device=x.device)
        else:
            idx, val, key = out
        lg = torch.empty((m, n), dtype=torch.bfloat16, device=x.device) if logits else None
        check(self._lib.qfg_lmhead_compute(self._h, x.data_ptr(), m, k, ctypes.byref(t), int(n), int(col_offset),
                                           self.workspace.data_ptr(), idx.data_ptr(), val.data_ptr(), key.data_ptr(),
                                           lg.data_ptr() if logits else None, _stream_ptr()))
        return (idx, val, key, lg) if logits else (idx, val, key)

    def call_sharded(self, x: torch.Tensor, w: torch.Tensor, n: int, col_offset: int, exchange, out=None):
        """qfg_lmhead_compute_sharded: this rank's columns, keys exchanged through the peers' memory inside
        the kernel; returns the node-wide (idx, val), identical on every rank.  `exchange` is an
        _lib.LmExchange whose buffers the caller set up (see lmhead_shard.PeerExchange)."""
        _require_cuda(x, "x")
        k = x.shape[-1]
        m = x.numel() // k
        t = _tensor2d(w)
        if out is None:
            out = (torch.empty(m, dtype=torch.int64, device=x.device), torch.empty(m, dtype=torch.float32, device=x.device))
        idx, val = out
        check(self._lib.qfg_lmhead_compute_sharded(self._h, x.data_ptr(), m, k, ctypes.byref(t), int(n), int(col_offset),
                                                   self.workspace.data_ptr(), ctypes.byref(exchange), idx.data_ptr(),
                                                   val.data_ptr(), None, _stream_ptr()))
        return idx, val

    def call_static(self, x: torch.Tensor, w: torch.Tensor, n: int, col_offset: int = 0, out=None):
        """The same computation through qfg_lmhead_compute_static: the scratch is the library's
        built-in array, nothing is taken from this instance's workspace.  `out` must be given by
        callers that may not allocate; at most 8 rows; calls must not overlap on one GPU."""
        _require_cuda(x, "x")
        k = x.shape[-1]
        m = x.numel() // k
        t = _tensor2d(w)
        if out is None:
            out = (torch.empty(m, dtype=torch.int64, device=x.device), torch.empty(m, dtype=torch.float32, device=x.device),
                   torch.empty(m, dtype=torch.int64, device=x.device))
        idx, val, key = out
        check(self._lib.qfg_lmhead_compute_static(self._h, x.data_ptr(), m, k, ctypes.byref(t), int(n), int(col_offset),
                                                  idx.data_ptr(), val.data_ptr(), key.data_ptr(), None, _stream_ptr()))
        return idx, val, key

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.qfg_lmhead_destroy(h)
            self._h = None


def lmhead_combine(keys: torch.Tensor, ranks: int, m: int):
    """Fold all-gathered keys [ranks, m] into (idx int64 [m], val float32 [m])."""
    lib = _lib.load()
    idx = torch.empty(m, dtype=torch.int64, device=keys.device)
    val = torch.empty(m, dtype=torch.float32, device=keys.device)
    check(lib.qfg_lmhead_combine(keys.data_ptr(), int(ranks), int(m), idx.data_ptr(), val.data_ptr(), _stream_ptr()))
    return idx, val
