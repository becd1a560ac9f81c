"""SharedExpertDown on the GPU: against the CPU oracle, the reference project's own kernel (when it was
compiled into oracle/_ref) and the decode-vs-chunks comparison of the reference's test
(tests/test_load.py:374-402)."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import bits, to_dev
from oracle import oracle as O
from qwen38_flash_ops_b200 import QfgError, SharedExpertDown
from qwen38_flash_ops_b200 import packing as P

import _util as U

pytestmark = pytest.mark.gpu


def _inputs(rng, M, K, N, gk):
    def bf(a):
        return P.f32_to_bf16_bits(a.astype(np.float32))
    g = bf(rng.standard_normal((M, K)) * 0.8)
    u = bf(rng.standard_normal((M, K)) * 0.8)
    gx = bf(rng.standard_normal((M, gk)) * 0.2)
    gw = bf(rng.standard_normal((gk, 1)) * 0.2)
    routed = bf(rng.standard_normal((M, N)) * 0.2)
    return g, u, gx, gw, routed


def _check(got, y, shared, routed_f, label):
    """Bit-exact except where an FP32 rounding difference (accumulation order, expf) crosses a BF16
    boundary: those may be one BF16 ULP of the larger of |routed| and |shared| off."""
    gf, yf = O.bf16_to_f32(got), O.bf16_to_f32(y)
    scale = np.maximum(np.maximum(np.abs(routed_f), np.abs(shared)), np.abs(yf))
    tol = scale * 2.0 ** -7 + 1e-30
    assert np.all(np.abs(gf - yf) <= tol), f"{label}: {np.count_nonzero(np.abs(gf - yf) > tol)} outputs outside one ULP"
    assert np.mean(got == y) > 0.97, f"{label}: only {np.mean(got == y):.4f} bit-exact"


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("M", [1, 2, 4, 7])
def test_against_oracle(cuda, mode, M):
    rng = np.random.default_rng(100 * mode + M)
    K, N, gk = 640, 1280, 1024
    arr, s = U.make_weight(rng, mode, K, N, mode != 0)
    g, u, gx, gw, routed = _inputs(rng, M, K, N, gk)
    op = SharedExpertDown(w_scale=s if mode != 0 else None)
    out = op(to_dev(g, "bf16"), to_dev(u, "bf16"), U.dev_weight(arr, mode), to_dev(gx, "bf16"), to_dev(gw, "bf16"),
             to_dev(routed, "bf16"))
    torch.cuda.synchronize()
    y, xb, gate, shared = O.shared_expert_down(g, u, mode, arr, N, gx, gw, routed, s if mode != 0 else None)
    _check(bits(out), y, shared, O.bf16_to_f32(routed), f"mode {mode} M {M}")


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_against_reference_kernel(cuda, mode):
    """The reference's GemvBody<FUSE> compiled for sm_100a with the launch configuration its operator uses."""
    lib = U.ref_lib()
    if lib is None or not hasattr(lib, "ref_shared_expert_down"):
        pytest.skip("reference kernels were not compiled")
    rng = np.random.default_rng(7 + mode)
    K, N, gk = 1024, 2048, 512
    for M in (1, 2, 4):
        arr, s = U.make_weight(rng, mode, K, N, mode != 0)
        g, u, gx, gw, routed = _inputs(rng, M, K, N, gk)
        dev = [to_dev(t, "bf16") for t in (g, u, gx, gw, routed)]
        w = U.dev_weight(arr, mode)
        op = SharedExpertDown(w_scale=s if mode != 0 else None)
        out = op(dev[0], dev[1], w, dev[2], dev[3], dev[4])
        ref = torch.empty_like(dev[4])
        sd = torch.tensor(s, dtype=torch.float32, device="cuda") if (mode != 0 and s is not None) else None
        err = lib.ref_shared_expert_down(ctypes.c_void_p(dev[0].data_ptr()), ctypes.c_void_p(dev[1].data_ptr()), M, K,
                                         ctypes.c_void_p(w.data_ptr()), mode, N,
                                         ctypes.c_void_p(sd.data_ptr() if sd is not None else None),
                                         ctypes.c_void_p(dev[2].data_ptr()), gk, ctypes.c_void_p(dev[3].data_ptr()),
                                         ctypes.c_void_p(dev[4].data_ptr()), ctypes.c_void_p(ref.data_ptr()), 0,
                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert err == 0
        torch.cuda.synchronize()
        a, b = bits(out).astype(np.int32), bits(ref).astype(np.int32)
        assert np.mean(a == b) > 0.97, f"mode {mode} M {M}: {np.mean(a == b):.4f} identical"
        y, xb, gate, shared = O.shared_expert_down(g, u, mode, arr, N, gx, gw, routed, s if mode != 0 else None)
        _check(bits(ref), y, shared, O.bf16_to_f32(routed), f"reference kernel vs oracle, mode {mode} M {M}")


def test_many_rows_match_two_row_chunks(cuda):
    """tests/test_load.py:374-402 of the reference: 16 rows in one call against eight 2-row calls
    (relative error < 0.002 there, where 16 rows take a dense prefill kernel; here both run the same
    kernel and the rows must be bit-identical)."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    K, N = 256, 128
    mk = lambda *s: (torch.randn(*s, generator=gen, device="cuda") * 0.2).bfloat16()
    g16, u16, gx16, gw, routed16 = mk(1, 16, K), mk(1, 16, K), mk(1, 16, K), mk(K, 1), mk(1, 16, N)
    wf = torch.randn(K, N, generator=gen, device="cuda") * 0.05
    sc = (wf.abs().amax(dim=0).clamp(min=1e-8) / 448.0).float()
    wq = (wf / sc[None, :]).clamp(-448, 448).to(torch.float8_e4m3fn)
    op = SharedExpertDown(w_scale=sc.cpu().numpy())
    full = op(g16, u16, wq, gx16, gw, routed16)
    parts = torch.cat([op(g16[:, i:i + 2].contiguous(), u16[:, i:i + 2].contiguous(), wq, gx16[:, i:i + 2].contiguous(), gw,
                          routed16[:, i:i + 2].contiguous()) for i in range(0, 16, 2)], dim=1)
    torch.cuda.synchronize()
    assert torch.equal(full, parts)
    rel = ((full.float() - parts.float()).norm() / parts.float().norm()).item()
    assert rel < 0.002


def test_argument_errors(cuda):
    op = SharedExpertDown()
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(QfgError):   # gk odd
        op(z(1, 64), z(1, 64), z(64, 64), z(1, 63), z(63, 1), z(1, 64))
    with pytest.raises(QfgError):   # N not a multiple of 8
        op(z(1, 64), z(1, 64), z(64, 60), z(1, 64), z(64, 1), z(1, 60))
    with pytest.raises(QfgError):   # routed rows do not match
        op(z(2, 64), z(2, 64), z(64, 64), z(2, 64), z(64, 1), z(1, 64))
