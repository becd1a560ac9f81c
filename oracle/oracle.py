"""CPU oracle (numpy) for the qwen.fused_gemm decode path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, the arithmetic of the reference's SkinnyGemm,
DequantWeightBf16 and ArgmaxRows kernels.  It is the checker that the tests, the smoke
entry and the benchmark's CPU-baseline leg compare the CUDA library against; nothing in the
shipped package imports it, and the product has no CPU code path.

Parity status.  The reference has no CPU implementation of this path, so each function
follows the CUDA source lines cited in its docstring (paths are inside the reference
project).  The restatement is pinned three ways:
  * against the formulas the reference's own op tests assert
    (tests/test_load.py:192-205 argmax with a planted tie, :322-342 FP8 dequantisation,
    :344-372 FP8 GEMM), re-expressed with torch on the CPU;
  * against ml_dtypes' float8_e4m3fn / float4_e2m1fn decode tables;
  * against outputs of the reference's kernel headers (src/fused_gemm/skinny_gemm.cuh,
    argmax_rows.cuh) compiled for sm_100a and run on a B200, stored as fixtures under
    tests/golden/ together with the script that generated them.
NVFP4 and BF16 SkinnyGemm have no test in the reference; for those the compiled kernels and
the cited source lines are the only pin.  DequantWeightBf16's kernel sits in the reference's ONNX
Runtime translation unit, which cannot be compiled without ONNX Runtime: its FP8 arithmetic is pinned by
the reference's own test formula, its NVFP4 arithmetic is PARITY UNPINNED by any reference output (held by
the cited source lines and the ml_dtypes tables only).

Conventions: BF16 / FP16 tensors travel as uint16 bit patterns, FP8 and packed NVFP4 as
uint8.  A packed NVFP4 row of an [K, N] weight is N/2 nibble bytes (column 2b in the low
nibble of byte b) followed by N/16 E4M3FN scale bytes, scale j covering columns
[16j, 16j+16) of that row (src/fused_gemm/skinny_gemm.cuh:200-204,
src/fused_gemm/fused_gemm.cu:220-223).
"""
from __future__ import annotations

import numpy as np

MODE_BF16, MODE_FP8, MODE_NVFP4 = 0, 1, 2


# ----------------------------------------------------------------------------- scalar formats
def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """BF16 bit patterns -> float32 (exact widening, skinny_gemm.cuh:106-109)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> BF16 bit patterns, round to nearest even (the `__float2bfloat16` of
    skinny_gemm.cuh:212).  NaN maps to the canonical quiet NaN 0x7FFF like the CUDA intrinsic."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounded = ((u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))) >> 16).astype(np.uint16)
    return np.where(np.isnan(x), np.uint16(0x7FFF), rounded)


def f16_to_f32(bits: np.ndarray) -> np.ndarray:
    """FP16 bits -> float32; a NaN becomes the canonical 0x7FFFFFFF that cvt.f32.f16 (the
    `__half2float` of argmax_rows.cuh:35) returns whatever the payload."""
    h = np.asarray(bits, dtype=np.uint16).view(np.float16)
    f = h.astype(np.float32)
    u = f.view(np.uint32).copy()
    u[np.isnan(h)] = 0x7FFFFFFF
    return u.view(np.float32)


def _e4m3fn_table() -> np.ndarray:
    """Decode table of the 256 E4M3FN codes (bias 7, no infinities, 0x7F/0xFF are NaN);
    the `__nv_cvt_fp8_to_halfraw(.., __NV_E4M3)` of skinny_gemm.cuh:112,169."""
    t = np.zeros(256, dtype=np.float32)
    for c in range(256):
        s = -1.0 if c & 0x80 else 1.0
        e = (c >> 3) & 0xF
        m = c & 7
        if e == 0xF and m == 7:
            v = np.nan
        elif e == 0:
            v = s * m * 2.0 ** -9
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[c] = v
    return t


E4M3 = _e4m3fn_table()
# 2 * |value| of the eight E2M1 magnitudes: the nibble LUT 0xC8643210 of skinny_gemm.cuh:162.
E2M1_MAG2 = np.array([0, 1, 2, 3, 4, 6, 8, 12], dtype=np.float32)


def e2m1_scaled(nib: np.ndarray, s_half: np.ndarray) -> np.ndarray:
    """`E2M1ScaledToFloat` (skinny_gemm.cuh:161-165): float(2*mag) * (scale/2), then the sign
    bit (nibble bit 3) is XOR-ed in, so nibble 0x8 is -0 and a NaN scale stays NaN."""
    f = E2M1_MAG2[nib & 7] * s_half
    return (f.view(np.uint32) ^ ((nib.astype(np.uint32) & 8) << 28)).view(np.float32)


# ----------------------------------------------------------------------------- weight decode
def nvfp4_unpack(packed: np.ndarray, n_cols_total: int):
    """Split a packed [K, 9N/16] tensor into nibbles [K, N] (uint8) and the half block scale
    [K, N/16] (float32 = E4M3(scale) * 0.5, skinny_gemm.cuh:169-170)."""
    packed = np.asarray(packed, dtype=np.uint8)
    K, cols = packed.shape
    N = n_cols_total
    assert N % 16 == 0 and cols == N * 9 // 16, "NVFP4 packed width must equal N * 9 / 16"
    nib_bytes = packed[:, : N // 2]
    nib = np.empty((K, N), dtype=np.uint8)
    nib[:, 0::2] = nib_bytes & 0xF
    nib[:, 1::2] = nib_bytes >> 4
    s_half = E4M3[packed[:, N // 2:]] * np.float32(0.5)
    return nib, s_half


def decode_weights_exact(mode: int, w: np.ndarray, n: int) -> np.ndarray:
    """The exact (unrounded) float32 value of every weight as the GEMV loop sees it:
    BF16 widen (skinny_gemm.cuh:106-109), E4M3 decode (:132-141), E2M1 x block scale
    (:167-175).  Every product E2M1 x E4M3 is exact in float32."""
    if mode == MODE_BF16:
        return bf16_to_f32(w)
    if mode == MODE_FP8:
        return E4M3[np.asarray(w, dtype=np.uint8)]
    nib, s_half = nvfp4_unpack(w, n)
    with np.errstate(invalid="ignore"):
        return e2m1_scaled(nib, np.repeat(s_half, 16, axis=1))


def dequant_weight_bf16(mode: int, w: np.ndarray, n_cols: int, col_offset: int = 0,
                        w_scale: np.ndarray | None = None) -> np.ndarray:
    """DequantWeightBf16 (fused_gemm.cu:203-250): a column slice [col_offset, col_offset+n_cols)
    of the weight as BF16 bits.  BF16: copy.  FP8: bf16_rn(float(q) * s[col]).  NVFP4:
    bf16_rn(E2M1Scaled * s[col]).  `w_scale` is indexed by OUTPUT column (:218, :226-227);
    without it the factor is 1."""
    if mode == MODE_BF16:
        return np.asarray(w, dtype=np.uint16)[:, col_offset:col_offset + n_cols].copy()
    if mode == MODE_FP8:
        vals = E4M3[np.asarray(w, dtype=np.uint8)[:, col_offset:col_offset + n_cols]]
    else:
        n_total = w.shape[1] * 16 // 9
        vals = decode_weights_exact(MODE_NVFP4, w, n_total)[:, col_offset:col_offset + n_cols]
    s = np.ones(n_cols, np.float32) if w_scale is None else np.asarray(w_scale, np.float32)[:n_cols]
    with np.errstate(invalid="ignore", over="ignore"):
        return f32_to_bf16(vals * s[None, :])


# ----------------------------------------------------------------------------- SkinnyGemm
def skinny_gemm(x_bits: np.ndarray, weights, seg_outs, widths, w_scale=None, col_block: int = 4096):
    """SkinnyGemm (fused_gemm.cu:507-592, skinny_gemm.cuh:332-536) with float64 accumulation.

    x_bits: [M, K] BF16 bits.  weights: list of (mode, array) per weight; BF16 [K,N] uint16,
    FP8 [K,N] uint8, NVFP4 [K,9N/16] uint8.  seg_outs[i] outputs slice weight i's columns,
    their widths listed in order in `widths`.  w_scale: float32 concatenation consumed by the
    quantised weights in order (fused_gemm.cu:553-556, :562-565); it multiplies the
    accumulated sum before the single BF16 rounding (skinny_gemm.cuh:228).

    Returns (outs, sums, mags): the BF16-bit outputs, and per weight the float64 sum (after
    w_scale) and sum of |x*w| (after |w_scale|), used for the robust tolerance
    |a-e| <= 2^-7 |e| + K 2^-24 sum|x w|.
    """
    x = bf16_to_f32(x_bits).astype(np.float64)
    M, K = x.shape
    outs, sums, mags = [], [], []
    o = 0
    scale_off = 0
    for i, (mode, w) in enumerate(weights):
        n = int(sum(widths[o:o + seg_outs[i]]))
        s = None
        if mode != MODE_BF16 and w_scale is not None and scale_off + n <= len(w_scale):
            s = np.asarray(w_scale[scale_off:scale_off + n], dtype=np.float32)
            scale_off += n
        acc = np.empty((M, n), dtype=np.float64)
        mag = np.empty((M, n), dtype=np.float64)
        for c0 in range(0, n, col_block):
            c1 = min(n, c0 + col_block)
            if mode == MODE_BF16:
                wv = bf16_to_f32(np.asarray(w)[:, c0:c1])
            elif mode == MODE_FP8:
                wv = E4M3[np.asarray(w, dtype=np.uint8)[:, c0:c1]]
            else:
                a0, a1 = (c0 // 16) * 16, -(-c1 // 16) * 16
                nibb = np.asarray(w, dtype=np.uint8)[:, a0 // 2:a1 // 2]
                nib = np.empty((K, a1 - a0), np.uint8)
                nib[:, 0::2] = nibb & 0xF
                nib[:, 1::2] = nibb >> 4
                sh = E4M3[np.asarray(w, dtype=np.uint8)[:, n // 2 + a0 // 16: n // 2 + a1 // 16]] * np.float32(0.5)
                with np.errstate(invalid="ignore"):
                    wv = e2m1_scaled(nib, np.repeat(sh, 16, axis=1))[:, c0 - a0:c1 - a0]
            wd = wv.astype(np.float64)
            with np.errstate(invalid="ignore"):
                acc[:, c0:c1] = x @ wd
                mag[:, c0:c1] = np.abs(x) @ np.abs(wd)
        if s is not None:
            with np.errstate(invalid="ignore", over="ignore"):
                y32 = acc.astype(np.float32) * s[None, :]
            acc = acc * s[None, :].astype(np.float64)
            mag = mag * np.abs(s[None, :]).astype(np.float64)
        else:
            with np.errstate(over="ignore"):
                y32 = acc.astype(np.float32)
        ybits = f32_to_bf16(y32)
        begin = 0
        for j in range(seg_outs[i]):
            outs.append(ybits[:, begin:begin + widths[o + j]].copy())
            begin += widths[o + j]
        o += seg_outs[i]
        sums.append(acc)
        mags.append(mag)
    return outs, sums, mags


def gemm_within_tolerance(actual_bits, expect_sum, expect_mag, K):
    """The stated GEMM bar: within one BF16 ULP (relative 2^-7) of the FP32-accumulated
    reference, plus the FP32 accumulation-order term K * 2^-24 * sum|x*w| that any
    FP32-accumulating implementation (the reference kernel included) is subject to."""
    a = bf16_to_f32(actual_bits).astype(np.float64)
    e = np.asarray(expect_sum, dtype=np.float64)
    tol = 2.0 ** -7 * np.abs(e) + K * 2.0 ** -24 * np.asarray(expect_mag) + 1e-30
    both_nan = np.isnan(a) & np.isnan(e)
    ok = (np.abs(a - e) <= tol) | both_nan
    return ok


# ----------------------------------------------------------------------------- ArgmaxRows
def better(av, ai, bv, bi) -> bool:
    """`Better` (argmax_rows.cuh:27-32): NaN beats non-NaN; among NaNs or equal values the
    lower index wins; -0 == +0."""
    if av != av:
        return (bv == bv) or ai < bi
    if bv != bv:
        return False
    return av > bv or (av == bv and ai < bi)


def argmax_rows(x: np.ndarray):
    """ArgmaxRows (argmax_rows.cuh:55-163, fused_gemm.cu:735-778): per row the index of the
    first maximum (numpy semantics: lowest index on ties, the first NaN wins over everything)
    and that value as float32.  `x` is a float32 array [rows, V] (widen BF16/FP16 first)."""
    x = np.asarray(x, dtype=np.float32)
    rows, V = x.shape
    idx = np.empty(rows, dtype=np.int64)
    val = np.empty(rows, dtype=np.float32)
    for r in range(rows):
        row = x[r]
        nan = np.isnan(row)
        if nan.any():
            i = int(np.argmax(nan))
        else:
            i = int(np.argmax(row))  # first maximum; -0.0 == +0.0 under IEEE comparison
        idx[r] = i
        val[r] = row[i]
    return idx, val


def combine_pairs(vals: np.ndarray, idxs: np.ndarray):
    """Combine per-shard (max, global index) pairs [shards, rows] with the `Better` order:
    the cross-rank step of the N-sharded LM head."""
    shards, rows = vals.shape
    out_i = np.empty(rows, dtype=np.int64)
    out_v = np.empty(rows, dtype=np.float32)
    for r in range(rows):
        bv, bi = np.float32(vals[0, r]), int(idxs[0, r])
        for s in range(1, shards):
            v, i = np.float32(vals[s, r]), int(idxs[s, r])
            if better(v, i, bv, bi):
                bv, bi = v, i
        out_i[r], out_v[r] = bi, bv
    return out_i, out_v


def lmhead_argmax(x_bits, mode, w, n, w_scale=None):
    """SkinnyGemm followed by ArgmaxRows over the BF16-rounded logits (the chain the fused
    LM-head entry point replaces).  Returns (idx, val, logits_bits, sums)."""
    outs, sums, mags = skinny_gemm(x_bits, [(mode, w)], [1], [n], w_scale)
    logits = outs[0]
    idx, val = argmax_rows(bf16_to_f32(logits))
    return idx, val, logits, sums[0]


# ----------------------------------------------------------------------------- UntileHcBf16
def untile_hc_bf16(w: np.ndarray, kind: int, fp8: bool, w_scale: np.ndarray | None = None) -> np.ndarray:
    """UntileHcBf16 (fused_gemm.cu:979-1011): the pre-tiled [160, 20480] tensor (uint16 BF16 bits, or
    uint8 E4M3FN codes when `fp8`) back to row-major BF16 bits, [10240, 320] (kind 0) or [320, 10240]
    (kind 1).  The tensor is 204800 groups of 16 consecutive elements and the op permutes groups:
    kind 0 reads group idx = ((s*20 + j)*10 + i)*128 + r and writes group ((s*10 + i)*128 + r)*20 + j
    (:985-993); kind 1 reads idx = ((h*10 + i)*32 + r)*4 + c and writes ((i*32 + r)*4 + c)*160 + h
    (:994-1003).  FP8 is dequantised with the scale of the OUTPUT column (:1008-1010)."""
    groups = np.asarray(w).reshape(204800, 16)
    idx = np.arange(204800)
    if kind == 0:
        r = idx & 127
        t1 = idx >> 7
        i = t1 % 10
        t2 = t1 // 10
        j = t2 % 20
        s = t2 // 20
        dst = ((s * 10 + i) * 128 + r) * 20 + j
        shape = (10240, 320)
    else:
        c = idx & 3
        t1 = idx >> 2
        r = t1 & 31
        t2 = t1 >> 5
        i = t2 % 10
        h = t2 // 10
        dst = ((i * 32 + r) * 4 + c) * 160 + h
        shape = (320, 10240)
    out_groups = np.empty_like(groups)
    out_groups[dst] = groups
    out = out_groups.reshape(shape)
    if not fp8:
        return out.astype(np.uint16)
    s = np.ones(shape[1], np.float32) if w_scale is None else np.asarray(w_scale, np.float32)[:shape[1]]
    with np.errstate(invalid="ignore", over="ignore"):
        return f32_to_bf16(E4M3[out.astype(np.uint8)] * s[None, :])


# ----------------------------------------------------------------------------- SharedExpertDown
def _round_bf16(v: np.ndarray) -> np.ndarray:
    """FP32 -> BF16 (RN) -> FP32: `Round` of skinny_gemm.cuh:73."""
    return bf16_to_f32(f32_to_bf16(np.asarray(v, np.float32)))


def sigmoid_bf16(a: np.ndarray) -> np.ndarray:
    """SigmoidBf16 of src/common/sigmoid_acc.cuh:12-18: e = exp(-|a|), 1/(1+e) for a > 0 else e/(1+e), in
    FP32, rounded once to BF16.  Evaluated in float64 here and rounded to FP32 first, which agrees with the
    device's expf except where the FP32 result sits on a BF16 rounding boundary."""
    a64 = np.asarray(a, np.float32).astype(np.float64)
    e = np.exp(-np.abs(a64))
    s = np.where(a64 > 0, 1.0 / (1.0 + e), e / (1.0 + e))
    return _round_bf16(s.astype(np.float32))


def swish_mul(g_bits: np.ndarray, u_bits: np.ndarray) -> np.ndarray:
    """SwishMulValue (skinny_gemm.cuh:77-80): bf16( bf16( g * bf16(sigmoid(g)) ) * u ), as BF16 bits."""
    g = bf16_to_f32(g_bits)
    u = bf16_to_f32(u_bits)
    swish = _round_bf16(g * sigmoid_bf16(g))
    return f32_to_bf16(swish * u)


def shared_expert_down(g_bits, u_bits, mode, w, n, gx_bits, gw_bits, routed_bits=None, w_scale=None):
    """SharedExpertDown (fused_gemm.cu:595; skinny_gemm.cuh:226-240, 302-327, 494-505):
    y = routed + bf16( bf16( swish_mul(g, u) @ W [* w_scale] ) * gate ),  gate = bf16(sigmoid(bf16(gx . gw))).
    The matrix product and the gate dot product are accumulated in float64 here (FP32 on the device, in
    kernel-dependent orders).  Returns (y bits, x' bits, gate, shared term before the routed add)."""
    x_bits = swish_mul(g_bits, u_bits)
    wf = decode_weights_exact(mode, w, n).astype(np.float64)
    acc = bf16_to_f32(x_bits).astype(np.float64) @ wf
    if w_scale is not None and mode != MODE_BF16:
        acc = acc * np.asarray(w_scale, np.float32)[:n].astype(np.float64)[None, :]
    logit = (bf16_to_f32(gx_bits).astype(np.float64) * bf16_to_f32(np.asarray(gw_bits).reshape(-1)).astype(np.float64)[None, :]).sum(axis=1)
    gate = sigmoid_bf16(_round_bf16(logit.astype(np.float32)))
    shared = _round_bf16(_round_bf16(acc.astype(np.float32)) * gate[:, None])
    if routed_bits is None:
        y = f32_to_bf16(shared)
    else:
        y = f32_to_bf16(bf16_to_f32(routed_bits) + shared)
    return y, x_bits, gate, shared
