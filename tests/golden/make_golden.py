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
    # SharedExpertDown: the reference's fused GEMV (its operator's launch configuration), one case per weight type
    import ctypes

    lib = U.ref_lib()
    if hasattr(lib, "ref_shared_expert_down"):
        for tag, mode, M, K, N, gk, scaled in (("bf16", 0, 1, 256, 128, 64, False), ("fp8", 1, 2, 320, 256, 128, True),
                                               ("nvfp4", 2, 4, 512, 128, 256, True)):
            rng = np.random.default_rng(40 + mode)
            bf = lambda a: P.f32_to_bf16_bits(a.astype(np.float32))
            g, u = bf(rng.standard_normal((M, K)) * 0.8), bf(rng.standard_normal((M, K)) * 0.8)
            gx, gw = bf(rng.standard_normal((M, gk)) * 0.2), bf(rng.standard_normal((gk, 1)) * 0.2)
            routed = bf(rng.standard_normal((M, N)) * 0.2)
            arr, s = U.make_weight(rng, mode, K, N, scaled)
            dev = [to_dev(t, "bf16") for t in (g, u, gx, gw, routed)]
            w = U.dev_weight(arr, mode)
            sd = torch.from_numpy(s).cuda() if s is not None else None
            out = torch.empty_like(dev[4])
            vp = ctypes.c_void_p
            err = lib.ref_shared_expert_down(vp(dev[0].data_ptr()), vp(dev[1].data_ptr()), M, K, vp(w.data_ptr()), mode, N,
                                             vp(sd.data_ptr() if sd is not None else None), vp(dev[2].data_ptr()), gk,
                                             vp(dev[3].data_ptr()), vp(dev[4].data_ptr()), vp(out.data_ptr()), 0,
                                             vp(torch.cuda.current_stream().cuda_stream))
            assert err == 0
            torch.cuda.synchronize()
            np.savez_compressed(os.path.join(out_dir, f"ref_shared_expert_down_{tag}.npz"), kind="shared_expert_down", mode=mode,
                                n=N, g=g, u=u, gx=gx, gw=gw, routed=routed, w=arr.view(np.uint8) if mode != 0 else arr,
                                w_scale=s if s is not None else np.zeros(0, np.float32), y=bits(out))
    print("wrote", sorted(os.listdir(out_dir)))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden"))
