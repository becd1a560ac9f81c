"""torch versions of the NVFP4 / FP8 packers, for generating large synthetic weights on the
GPU (the numpy packers in packing.py are the definition; tests check that these agree)."""
from __future__ import annotations

import torch

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# decision boundaries between consecutive magnitudes; a tie goes to the even code
_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_TIE_TO_LOWER = (True, False, True, False, True, False, True)  # lower code of each pair is even at pairs 0,2,4,6


def e2m1_encode_torch(x: torch.Tensor) -> torch.Tensor:
    a = x.abs().clamp(max=6.0)
    code = torch.zeros_like(a, dtype=torch.uint8)
    for b, lower in zip(_BOUNDS, _TIE_TO_LOWER):
        code += ((a > b) if lower else (a >= b)).to(torch.uint8)
    return code | (torch.signbit(x).to(torch.uint8) << 3)


def pack_nvfp4_torch(w: torch.Tensor) -> torch.Tensor:
    """[K, N] float32 -> UINT8 [K, N*9/16] in the [nibbles | block scales] row layout."""
    K, N = w.shape
    assert N % 16 == 0
    blocks = w.float().reshape(K, N // 16, 16)
    amax = blocks.abs().amax(dim=2)
    sc = (amax / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    scode = sc.view(torch.uint8)
    scode = torch.where(scode == 0, torch.ones_like(scode), scode)
    s = scode.view(torch.float8_e4m3fn).float()
    nib = e2m1_encode_torch((blocks.double() / s.double()[:, :, None]).float() if False else blocks / s[:, :, None])
    nib = nib.reshape(K, N)
    out = torch.empty((K, N * 9 // 16), dtype=torch.uint8, device=w.device)
    out[:, : N // 2] = nib[:, 0::2] | (nib[:, 1::2] << 4)
    out[:, N // 2:] = scode
    return out


def quantize_fp8_per_column_torch(w: torch.Tensor):
    amax = w.float().abs().amax(dim=0).clamp(min=1e-8)
    s = (amax / 448.0).float()
    q = (w.float() / s[None, :]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q, s
