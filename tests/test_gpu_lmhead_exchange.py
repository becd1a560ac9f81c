"""The in-kernel key exchange of the N-sharded LM head (qfg_lmhead_compute_sharded) on ONE GPU.

Two ranks are emulated as two calls, one after the other, whose exchange buffers both live on this
device.  The rank that runs first stores its words into both buffers, finds nobody else's, and its
bounded wait runs out (short limit): status 1, result = its own winner.  The rank that runs second
finds the first rank's words already there: status 0, and its result must equal the single-GPU fused
head over the whole vocabulary, bit for bit.  Nothing here needs two kernels to run at the same time;
what only concurrent ranks can show (both waits completing) is checked by bench.py on 2-8 GPUs.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import to_dev
from qwen38_flash_ops_b200 import LmHeadArgmax, QfgError, _lib
from qwen38_flash_ops_b200 import packing as P
from qwen38_flash_ops_b200.ops import _tensor2d

import _util as U

pytestmark = pytest.mark.gpu


class TwoRanks:
    """Two exchange buffers on one device and one fused head per emulated rank."""

    def __init__(self, spin_first=64):
        lib = _lib.load()
        nbytes = lib.qfg_lmhead_exchange_bytes()
        self.bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
        self.heads = [LmHeadArgmax(), LmHeadArgmax()]
        self.ex = []
        for r in range(2):
            e = _lib.LmExchange()
            e.world, e.rank = 2, r
            for q in range(2):
                e.peers[q] = self.bufs[q].data_ptr()
            self.ex.append(e)
        self.spin_first = spin_first
        self.lib = lib

    def status(self, r):
        s = ctypes.c_int(-1)
        _lib.check(self.lib.qfg_lmhead_exchange_status(self.bufs[r].data_ptr(), ctypes.byref(s)))
        return s.value

    def clear_status(self, r):
        # status is the second 32-bit word after the 2048 bytes of slots and the call count
        self.bufs[r].view(torch.int32)[2048 // 4 + 1] = 0

    def step(self, x, shards, widths, offsets, first):
        """Runs rank `first` (short wait limit), then the other rank.  Returns their (idx, val) pairs."""
        out = [None, None]
        for r, spin in ((first, self.spin_first), (1 - first, 1 << 22)):
            self.heads[r].set_option("exchange_spin", spin)
            out[r] = self.heads[r].call_sharded(x, shards[r], widths[r], offsets[r], self.ex[r])
            torch.cuda.synchronize()
        return out


def _split(arr, mode, n, c_mid):
    if mode == 2:
        return [P.nvfp4_column_slice(arr, n, 0, c_mid), P.nvfp4_column_slice(arr, n, c_mid, n)]
    return [np.ascontiguousarray(arr[:, :c_mid]), np.ascontiguousarray(arr[:, c_mid:])]


@pytest.mark.parametrize("mode", [0, 2])
def test_second_rank_folds_the_first_and_equals_the_single_gpu_head(cuda, mode):
    rng = np.random.default_rng(900 + mode)
    K, N, c_mid = 512, 128 * 26, 128 * 15
    arr, _ = U.make_weight(rng, mode, K, N, False)
    whole = U.dev_weight(arr, mode)
    parts = [U.dev_weight(a, mode) for a in _split(arr, mode, N, c_mid)]
    widths, offsets = [c_mid, N - c_mid], [0, c_mid]
    tr = TwoRanks()
    single = LmHeadArgmax()
    first = 1
    for call, m in enumerate((1, 2, 4, 8, 3, 4)):   # consecutive calls alternate the slot parity
        x = to_dev(P.synth_x(rng, m, K), "bf16")
        ref_idx, ref_val, _ = single(x, whole, N)
        own = [single(x, parts[r], widths[r], col_offset=offsets[r]) for r in range(2)]
        out = tr.step(x, parts, widths, offsets, first)
        # the first rank gave up on its peer: it reports that, and its result is its own shard's winner
        assert tr.status(first) == 1, f"call {call}"
        assert torch.equal(out[first][0], own[first][0]) and torch.equal(out[first][1], own[first][1])
        # the second rank found everything: clean status and the single-GPU result
        assert tr.status(1 - first) == 0, f"call {call}"
        assert torch.equal(out[1 - first][0], ref_idx), f"call {call}, m {m}"
        assert torch.equal(out[1 - first][1].view(torch.int32), ref_val.view(torch.int32))
        tr.clear_status(first)
        first = 1 - first   # both orders, both parities
        for h in tr.heads:  # the workspaces come back clean
            assert int(h.workspace.view(torch.int64).abs().sum().item()) == 0


def test_cross_shard_tie_and_nan(cuda):
    K, N, c_mid = 256, 2048, 1024
    w = np.zeros((K, N), np.float32)
    w[0, 300] = w[0, 1700] = 0.5            # equal maxima in different shards: the lower global index wins
    x = np.zeros((2, K), np.float32)
    x[0, 0] = 2.0
    x[1, 0] = -1.0                          # row 1: every logit <= 0, the maximum 0 first at column 0
    xd = to_dev(P.f32_to_bf16_bits(x), "bf16")
    for nan_cols, expect in (((), [300, 0]), ((1500,), [1500, 1500]), ((1500, 100), [100, 100])):
        wn = w.copy()
        for c in nan_cols:
            wn[0, c] = np.nan
        bits = P.f32_to_bf16_bits(wn)
        parts = [U.dev_weight(a, 0) for a in _split(bits, 0, N, c_mid)]
        for first in (0, 1):
            tr = TwoRanks()
            out = tr.step(xd, parts, [c_mid, N - c_mid], [0, c_mid], first)
            idx, val = out[1 - first]
            assert idx.tolist() == expect, (nan_cols, first)
            if nan_cols:
                assert bool(torch.isnan(val).all())
            else:
                assert val.tolist() == [1.0, 0.0]
            assert tr.status(1 - first) == 0 and tr.status(first) == 1


def test_host_step_fails_when_a_peer_never_arrives(cuda):
    """qfg_lmhead_host_run reads the per-step status word and returns QFG_FAIL instead of a partial result."""
    rng = np.random.default_rng(5)
    K, N, m = 256, 1024, 2
    pk = to_dev(P.pack_nvfp4(P.synth_weight(rng, K, N)), "u8")
    tr = TwoRanks()
    head = tr.heads[1]
    head.set_option("exchange_spin", 64)
    lib = tr.lib
    x_host = torch.zeros((m, K), dtype=torch.bfloat16).pin_memory()
    x_dev = torch.zeros((m, K), dtype=torch.bfloat16, device="cuda")
    idx_host = torch.zeros(m, dtype=torch.int64).pin_memory()
    val_host = torch.zeros(m, dtype=torch.float32).pin_memory()
    t = _tensor2d(pk)
    h = ctypes.c_void_p()
    torch.cuda.synchronize()
    _lib.check(lib.qfg_lmhead_host_create(head._h, m, K, ctypes.byref(t), N, 512, head.workspace.data_ptr(),
                                          ctypes.byref(tr.ex[1]), x_host.data_ptr(), x_dev.data_ptr(),
                                          idx_host.data_ptr(), val_host.data_ptr(), ctypes.byref(h)))
    try:
        rc = lib.qfg_lmhead_host_run(h)
        assert rc == _lib.QFG_FAIL
        assert "ran out" in lib.qfg_last_error().decode()
        assert tr.status(1) == 1
    finally:
        lib.qfg_lmhead_host_destroy(h)
