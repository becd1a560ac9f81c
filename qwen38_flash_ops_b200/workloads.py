"""The benchmark workloads: seeded synthetic stand-ins for the decode projections of the model the
reference serves (shapes, sizes and value distributions as the benchmark configuration names
them; no dataset or checkpoint is involved).  Weights are generated and packed on the GPU."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import packing_torch as PT

MODE_BF16, MODE_FP8, MODE_NVFP4 = 0, 1, 2


@dataclass
class Workload:
    name: str
    mode: int
    m: int
    k: int
    seg_widths: list          # per weight: list of output widths
    trigger: int = 0
    fused_argmax: bool = False
    notes: str = ""

    @property
    def ns(self):
        return [sum(w) for w in self.seg_widths]

    @property
    def weight_bytes(self) -> int:
        n = sum(self.ns)
        return {0: 2 * self.k * n, 1: self.k * n, 2: self.k * n * 9 // 16}[self.mode]

    def other_bytes(self) -> int:
        n = sum(self.ns)
        out = 12 * self.m if self.fused_argmax else 2 * self.m * n
        return (4 * n if self.mode == 1 else 0) + 2 * self.m * self.k + out


CONFIGS = {
    "C1_bf16_5120x5120": Workload("C1_bf16_5120x5120", MODE_BF16, 1, 5120, [[5120]]),
    "C2_fp8_qkv_5120x10240": Workload("C2_fp8_qkv_5120x10240", MODE_FP8, 2, 5120, [[8192], [1024], [1024]]),
    "C3_nvfp4_gate_up_5120x34816": Workload("C3_nvfp4_gate_up_5120x34816", MODE_NVFP4, 1, 5120, [[17408], [17408]]),
    "C4_nvfp4_down_17408x5120": Workload("C4_nvfp4_down_17408x5120", MODE_NVFP4, 4, 17408, [[5120]], trigger=2),
    "C5_nvfp4_lmhead_5120x151936": Workload("C5_nvfp4_lmhead_5120x151936", MODE_NVFP4, 4, 5120, [[151936]],
                                            fused_argmax=True),
}


def make_x(m: int, k: int, seed: int, device="cuda") -> torch.Tensor:
    gen = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(m, k, generator=gen, device=device).bfloat16()


def make_weight(mode: int, k: int, n: int, seed: int, device="cuda", col_block: int = 32768):
    """One weight: (stored tensor, per-column scale tensor or None).  Source values ~ N(0, 0.02^2);
    FP8: s_col = amax_col / 448; NVFP4: block-16 scales E4M3(amax / 6)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    if mode == MODE_BF16:
        return (torch.randn(k, n, generator=gen, device=device) * 0.02).bfloat16(), None
    if mode == MODE_FP8:
        q, s = PT.quantize_fp8_per_column_torch(torch.randn(k, n, generator=gen, device=device) * 0.02)
        return q, s
    out = torch.empty((k, n * 9 // 16), dtype=torch.uint8, device=device)
    for c0 in range(0, n, col_block):
        c1 = min(n, c0 + col_block)
        blk = PT.pack_nvfp4_torch(torch.randn(k, c1 - c0, generator=gen, device=device) * 0.02)
        out[:, c0 // 2:c1 // 2] = blk[:, :(c1 - c0) // 2]
        out[:, n // 2 + c0 // 16:n // 2 + c1 // 16] = blk[:, (c1 - c0) // 2:]
    return out, None
