"""Shared helpers of the GPU parity tests: seeded workloads, oracle comparison, reference-kernel access."""
import ctypes
import os

import numpy as np

from oracle import cpu as C
from oracle import oracle as O
from qwen38_flash_ops_b200 import packing as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so")


def make_weight(rng, mode, K, N, with_scale=None):
    """Returns (stored array, w_scale or None) for one weight of the given mode."""
    w = P.synth_weight(rng, K, N)
    if mode == 0:
        return P.f32_to_bf16_bits(w), None
    if mode == 1:
        q, s = P.quantize_fp8_per_column(w)
        return q, (s if with_scale is not False else None)
    pk = P.pack_nvfp4(w)
    s = rng.uniform(0.5, 2.0, N).astype(np.float32) if with_scale else None
    return pk, s


def dev_weight(arr, mode):
    from conftest import to_dev

    return to_dev(arr, ["bf16", "fp8", "u8"][mode])


def check_against_oracle(mode, x_bits, w_arr, n, scale, got_bits, K, label=""):
    out, sums, mags = C.skinny_gemm(mode, x_bits, w_arr, n, scale)
    ok = O.gemm_within_tolerance(got_bits, sums, mags, K)
    assert ok.all(), f"{label}: {np.count_nonzero(~ok)} of {ok.size} outputs outside tolerance"
    # the literal one-BF16-ULP criterion on outputs that do not cancel
    e = sums
    a = O.bf16_to_f32(got_bits).astype(np.float64)
    big = np.abs(e) >= 2.0 ** -6 * np.sqrt(np.mean(e ** 2) + 1e-300)
    if big.any():
        lit = np.abs(a - e)[big] <= 2.0 ** -7 * np.abs(e)[big] + 1e-30
        assert lit.all(), f"{label}: literal 2^-7 criterion failed on {np.count_nonzero(~lit)} outputs"
    exact = np.mean(out == got_bits)
    return exact


_ref = None


def ref_lib():
    """The reference project's kernels compiled for sm_100a (absent if never built)."""
    global _ref
    if _ref is None:
        if not os.path.exists(REF_LIB):
            return None
        lib = ctypes.CDLL(REF_LIB)
        vp = ctypes.c_void_p
        lib.ref_skinny_gemm.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(vp),
                                        ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                        ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(vp),
                                        ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int, vp]
        lib.ref_argmax_rows.argtypes = [ctypes.c_int, vp, ctypes.c_longlong, ctypes.c_longlong, vp, vp, vp]
        if hasattr(lib, "ref_shared_expert_down"):
            ci = ctypes.c_int
            lib.ref_shared_expert_down.argtypes = [vp, vp, ci, ci, vp, ci, ci, vp, vp, ci, vp, vp, vp, ci, vp]
        _ref = lib
    return _ref


def ref_skinny_gemm(x, weights, modes, ns, scales, seg_outs, widths, trigger=0, cluster=0):
    """x: CUDA BF16 [m, k]; weights: CUDA tensors; scales: CUDA float tensors or None. Returns outputs."""
    import torch

    lib = ref_lib()
    m, k = x.shape
    nseg = len(weights)
    vp = ctypes.c_void_p
    outs = [torch.empty((m, w), dtype=torch.bfloat16, device=x.device) for w in widths]
    w_arr = (vp * nseg)(*[w.data_ptr() for w in weights])
    mode_arr = (ctypes.c_int * nseg)(*modes)
    n_arr = (ctypes.c_int * nseg)(*ns)
    s_arr = (vp * nseg)(*[(s.data_ptr() if s is not None else None) for s in scales])
    so_arr = (ctypes.c_int * nseg)(*seg_outs)
    o_arr = (vp * len(outs))(*[o.data_ptr() for o in outs])
    wd_arr = (ctypes.c_int * len(widths))(*widths)
    err = lib.ref_skinny_gemm(x.data_ptr(), m, k, nseg, w_arr, mode_arr, n_arr, s_arr, so_arr, o_arr, wd_arr,
                              trigger, cluster, torch.cuda.current_stream().cuda_stream)
    assert err == 0, f"reference kernel launch failed with cudaError {err}"
    return outs


def ref_argmax_rows(x):
    import torch

    lib = ref_lib()
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[x.dtype]
    rows, v = x.shape
    idx = torch.empty(rows, dtype=torch.int64, device=x.device)
    val = torch.empty(rows, dtype=torch.float32, device=x.device)
    err = lib.ref_argmax_rows(code, x.data_ptr(), rows, v, idx.data_ptr(), val.data_ptr(),
                              torch.cuda.current_stream().cuda_stream)
    assert err == 0
    return idx, val
