#!/usr/bin/env python3
"""Generates the golden fixtures of tests/golden/ref_*.npz.

Runs the reference project's own kernels (src/fused_gemm/skinny_gemm.cuh and argmax_rows.cuh,
compiled for sm_100a into oracle/_ref/libref_kernels.so by `make -C oracle`) on seeded inputs on
a B200 and stores inputs and outputs.  The fixtures pin the CPU oracle in the CPU-only test
suite (tests/test_oracle_cpu.py::test_golden_fixtures_from_reference_kernels).

    python tests/golden/make_golden.py <output directory>
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import _util as U  # noqa: E402
from conftest import bits, to_dev  # noqa: E402
from qwen38_flash_ops_b200 import packing as P  # noqa: E402


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    assert U.ref_lib() is not None, "build oracle/_ref first"
    # ArgmaxRows: the reference test's shape (rows 5, vocabulary 4099, planted tie) and a vector-path shape
    for tag, dtype, code, vocab in (("bf16_4099", torch.bfloat16, 0, 4099), ("f32_4099", torch.float32, 2, 4099),
                                    ("f16_4096", torch.float16, 1, 4096)):
        g = torch.Generator().manual_seed(3)
        x = torch.randn(5, vocab, generator=g).to(dtype)
        x[1, 17] = x[1, 3000] = x.max() + 1
        x[3, 11] = float("nan")
        x[3, 2000] = float("nan")
        x[4, :] = 0.0
        x[4, 7] = -0.0
        xd = x.cuda()
        idx, val = U.ref_argmax_rows(xd)
        torch.cuda.synchronize()
        raw = x.numpy() if code == 2 else x.view(torch.int16).numpy().view(np.uint16)
        np.savez_compressed(os.path.join(out_dir, f"ref_argmax_{tag}.npz"), kind="argmax", dtype_code=code, x=raw,
                            idx=idx.cpu().numpy(), val=val.cpu().numpy())
    # SkinnyGemm: one small case per weight type
    for tag, mode, M, K, N, scaled in (("bf16", 0, 1, 256, 64, False), ("fp8", 1, 2, 256, 128, True),
                                       ("nvfp4", 2, 4, 256, 128, False), ("nvfp4_scaled", 2, 3, 272, 192, True)):
        rng = np.random.default_rng(5 + mode + M)
        x = P.synth_x(rng, M, K)
        arr, s = U.make_weight(rng, mode, K, N, scaled)
        sd = torch.from_numpy(s).cuda() if s is not None else None
        y = U.ref_skinny_gemm(to_dev(x, "bf16"), [U.dev_weight(arr, mode)], [mode], [N], [sd], [1], [N])[0]
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, f"ref_gemm_{tag}.npz"), kind="gemm", mode=mode, n=N, x=x,
                            w=arr.view(np.uint8) if mode != 0 else arr, y=bits(y),
                            w_scale=s if s is not None else np.zeros(0, np.float32))
    print("wrote", sorted(os.listdir(out_dir)))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "gpurun_out", "golden"))
