"""Host-side weight packing for the three weight formats SkinnyGemm accepts.

These are the offline tools a model exporter needs: the per-column FP8 E4M3FN quantiser,
the block-16 NVFP4 packer that emits the `UINT8 [K, N*9/16]` row layout the kernels read,
and the column re-packer that cuts an NVFP4 tensor into per-rank shards for the N-sharded
LM head.  Pure numpy; nothing here runs on the decode path.

NVFP4 row layout (one row of a [K, N] weight): N/2 nibble bytes, column 2b in the low
nibble and column 2b+1 in the high nibble of byte b, followed by N/16 E4M3FN scale bytes;
scale j covers columns [16j, 16j+16) of the same row.  This is the layout the reference
reads at src/fused_gemm/skinny_gemm.cuh:200-204 and src/fused_gemm/fused_gemm.cu:220-223.
"""
from __future__ import annotations

import numpy as np

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def _e4m3_positive_table() -> np.ndarray:
    t = np.empty(127, dtype=np.float64)  # codes 0x00..0x7E (0x7F is NaN)
    for c in range(127):
        e, m = c >> 3, c & 7
        t[c] = m * 2.0 ** -9 if e == 0 else (1.0 + m / 8.0) * 2.0 ** (e - 7)
    return t


_E4M3_POS = _e4m3_positive_table()


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> BF16 bit patterns (uint16), round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))) >> 16).astype(np.uint16)
    return np.where(np.isnan(x), np.uint16(0x7FFF), r)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Round float values to the nearest E4M3FN code (ties to the even code), saturating at
    +-448.  NaN encodes as 0x7F."""
    x = np.asarray(x, dtype=np.float64)
    a = np.minimum(np.abs(x), 448.0)
    hi = np.searchsorted(_E4M3_POS, a, side="left").clip(0, 126)
    lo = (hi - 1).clip(0, 126)
    d_hi = np.abs(_E4M3_POS[hi] - a)
    d_lo = np.abs(a - _E4M3_POS[lo])
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & (lo % 2 == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    code = np.where(np.signbit(x), code | 0x80, code).astype(np.uint8)
    return np.where(np.isnan(x), np.uint8(0x7F), code)


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    code = np.asarray(code, dtype=np.uint8)
    mag = np.where((code & 0x7F) == 0x7F, np.nan, _E4M3_POS[np.minimum(code & 0x7F, 126)])
    return np.where(code & 0x80, -mag, mag).astype(np.float32)


def quantize_fp8_per_column(w: np.ndarray):
    """Per-column FP8: s_col = amax_col / 448 (float32), q = E4M3FN_RN(clamp(w / s_col, +-448)).
    Returns (q uint8 [K, N], s_col float32 [N])."""
    w = np.asarray(w, dtype=np.float32)
    amax = np.maximum(np.abs(w).max(axis=0), np.float32(1e-8))
    s = (amax / np.float32(448.0)).astype(np.float32)
    q = e4m3_encode(np.clip(w / s[None, :], -448.0, 448.0))
    return q, s


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """Nearest E2M1 code (sign | 3-bit magnitude index), ties to the even code, saturating at 6."""
    x = np.asarray(x, dtype=np.float64)
    a = np.minimum(np.abs(x), 6.0)
    v = E2M1_VALUES.astype(np.float64)
    hi = np.searchsorted(v, a, side="left").clip(0, 7)
    lo = (hi - 1).clip(0, 7)
    d_hi, d_lo = np.abs(v[hi] - a), np.abs(a - v[lo])
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & (lo % 2 == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    return np.where(np.signbit(x), code | 8, code).astype(np.uint8)


def pack_nvfp4(w: np.ndarray) -> np.ndarray:
    """Block-16 NVFP4: for each row and each group of 16 consecutive columns the scale is
    E4M3FN_RN(amax / 6) (code 0x01 if that rounds to zero), the nibbles are the nearest E2M1
    of w / scale.  Returns the UINT8 [K, N*9/16] tensor in the row layout described above."""
    w = np.asarray(w, dtype=np.float32)
    K, N = w.shape
    assert N % 16 == 0, "NVFP4 needs N % 16 == 0"
    blocks = w.reshape(K, N // 16, 16)
    amax = np.abs(blocks).max(axis=2)
    scode = e4m3_encode(amax / 6.0)
    scode = np.where(scode == 0, np.uint8(1), scode).astype(np.uint8)
    s = e4m3_decode(scode).astype(np.float64)
    nib = e2m1_encode(blocks / s[:, :, None]).reshape(K, N)
    out = np.empty((K, N * 9 // 16), dtype=np.uint8)
    out[:, : N // 2] = nib[:, 0::2] | (nib[:, 1::2] << 4)
    out[:, N // 2:] = scode
    return out


def nvfp4_column_slice(packed: np.ndarray, n_total: int, col_begin: int, col_end: int) -> np.ndarray:
    """Cut columns [col_begin, col_end) (multiples of 16) out of a packed NVFP4 tensor and
    re-pack them as a self-contained [K, 9*(col_end-col_begin)/16] tensor.  A column shard is
    not a contiguous slice of the packed rows, because each row is [nibbles | scales]."""
    assert col_begin % 16 == 0 and col_end % 16 == 0 and 0 <= col_begin < col_end <= n_total
    packed = np.asarray(packed, dtype=np.uint8)
    K = packed.shape[0]
    n = col_end - col_begin
    out = np.empty((K, n * 9 // 16), dtype=np.uint8)
    out[:, : n // 2] = packed[:, col_begin // 2: col_end // 2]
    out[:, n // 2:] = packed[:, n_total // 2 + col_begin // 16: n_total // 2 + col_end // 16]
    return out


def shard_columns(n_total: int, world: int, granule: int = 128):
    """Column ranges of an N-sharded LM head: granules of `granule` columns dealt out so that
    the first (n_granules % world) ranks hold one granule more.  128-column granules keep each
    rank's packed NVFP4 row pitch (9 * N_r / 16 bytes) a multiple of 8 bytes."""
    assert n_total % granule == 0, "vocabulary must be a multiple of the shard granule"
    g = n_total // granule
    base, extra = divmod(g, world)
    bounds, c = [], 0
    for r in range(world):
        w = (base + (1 if r < extra else 0)) * granule
        bounds.append((c, c + w))
        c += w
    return bounds


# ------------------------------------------------------------------ seeded synthetic workloads
def synth_x(rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    """Activations: BF16 bits of N(0, 1), shape [m, k]."""
    return f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))


def synth_weight(rng: np.random.Generator, k: int, n: int, sigma: float = 0.02) -> np.ndarray:
    return (rng.standard_normal((k, n), dtype=np.float32) * np.float32(sigma)).astype(np.float32)
