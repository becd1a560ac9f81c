import numpy as np
import torch

from oracle import oracle as O
from qwen38_flash_ops_b200 import packing as P
from qwen38_flash_ops_b200 import packing_torch as PT


def test_nvfp4_pack_layout_and_roundtrip():
    rng = np.random.default_rng(0)
    K, N = 8, 128
    w = P.synth_weight(rng, K, N)
    pk = P.pack_nvfp4(w)
    assert pk.shape == (K, N * 9 // 16)
    vals = O.decode_weights_exact(2, pk, N)
    # every block's dequantised maximum is within one E4M3 step of the source maximum,
    # and every weight within a coarse quantisation step of its block (scales are E4M3 subnormals here)
    s = O.E4M3[pk[:, N // 2:]]
    assert np.all(s > 0)
    err = np.abs(vals - w).reshape(K, N // 16, 16).max(axis=2)
    assert np.all(err <= s * 2.0 + 1e-9)
    # even column in the low nibble
    b0 = pk[0, 0]
    assert O.e2m1_scaled(np.array([b0 & 0xF], np.uint8), np.array([s[0, 0] * 0.5], np.float32))[0] == vals[0, 0]
    assert O.e2m1_scaled(np.array([b0 >> 4], np.uint8), np.array([s[0, 0] * 0.5], np.float32))[0] == vals[0, 1]


def test_column_slice_repack_equals_dequant_slice():
    rng = np.random.default_rng(1)
    K, N = 16, 512
    pk = P.pack_nvfp4(P.synth_weight(rng, K, N))
    full = O.decode_weights_exact(2, pk, N)
    for c0, c1 in ((0, 128), (128, 384), (384, 512)):
        shard = P.nvfp4_column_slice(pk, N, c0, c1)
        assert shard.shape == (K, (c1 - c0) * 9 // 16)
        assert np.array_equal(O.decode_weights_exact(2, shard, c1 - c0), full[:, c0:c1])


def test_shard_columns_partition():
    n = 151936
    for world in (1, 2, 4, 8):
        b = P.shard_columns(n, world)
        assert b[0][0] == 0 and b[-1][1] == n
        assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
        widths = [hi - lo for lo, hi in b]
        assert all(w % 128 == 0 for w in widths) and max(widths) - min(widths) <= 128
        assert all((w * 9 // 16) % 8 == 0 for w in widths)  # packed row pitch stays 8-byte aligned
    assert [hi - lo for lo, hi in P.shard_columns(n, 8)] == [19072] * 3 + [18944] * 5


def test_torch_packers_match_numpy():
    rng = np.random.default_rng(2)
    w = P.synth_weight(rng, 32, 256)
    assert np.array_equal(PT.pack_nvfp4_torch(torch.from_numpy(w)).numpy(), P.pack_nvfp4(w))
    q, s = PT.quantize_fp8_per_column_torch(torch.from_numpy(w))
    qn, sn = P.quantize_fp8_per_column(w)
    assert np.array_equal(s.numpy(), sn)
    assert np.array_equal(q.view(torch.uint8).numpy(), qn)
