"""GPU parity of ArgmaxRows and DequantWeightBf16 through the C ABI: bit-exact against the oracle."""
import numpy as np
import pytest
import torch

from conftest import bits, to_dev
from oracle import cpu as C
from oracle import oracle as O
from qwen38_flash_ops_b200 import ArgmaxRows, DequantWeightBf16, QfgError
from qwen38_flash_ops_b200 import packing as P

import _util as U

pytestmark = pytest.mark.gpu


def _check_argmax(x: torch.Tensor):
    idx, val = ArgmaxRows()(x)
    torch.cuda.synchronize()
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[x.dtype]
    raw = x.cpu().numpy() if code == 2 else bits(x)
    raw = raw.reshape(-1, x.shape[-1])
    eidx, eval_ = C.argmax_rows(code, raw)
    assert np.array_equal(idx.cpu().numpy().reshape(-1), eidx)
    assert np.array_equal(val.cpu().numpy().reshape(-1).view(np.uint32), eval_.view(np.uint32))
    if U.ref_lib() is not None and x.dim() == 2:
        ridx, rval = U.ref_argmax_rows(x)
        torch.cuda.synchronize()
        assert torch.equal(ridx, idx) and torch.equal(rval.view(torch.int32), val.view(torch.int32))
    return idx, val


def test_argmax_reference_test_case(cuda):
    # the reference's op test: rows 5, V 4099 (odd), BF16 and FP32, a planted tie must return 17
    rows, vocab = 5, 4099
    gen = torch.Generator(device="cuda").manual_seed(3)
    for dtype in (torch.bfloat16, torch.float32, torch.float16):
        x = torch.randn(rows, vocab, generator=gen, device="cuda").to(dtype)
        x[1, 17] = x[1, 3000] = x.max() + 1
        idx, val = _check_argmax(x)
        assert idx[1].item() == 17
        mx = x.float().max(dim=1)
        keep = torch.tensor([r != 1 for r in range(rows)], device="cuda")
        assert torch.equal(idx[keep], mx.indices[keep])
        assert torch.equal(val, mx.values)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("vocab", [1, 7, 8, 33, 1000, 151936, 248320])
def test_argmax_sizes(cuda, dtype, vocab):
    gen = torch.Generator(device="cuda").manual_seed(vocab)
    x = torch.randn(3, vocab, generator=gen, device="cuda").to(dtype)
    _check_argmax(x)


def test_argmax_special_values(cuda):
    V = 5000
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        x = torch.zeros(6, V, dtype=dtype, device="cuda")
        x[0, 4000] = -0.0                                  # all +-0: index 0
        x[1, 4100] = float("nan")
        x[1, 77] = float("nan")
        x[1, 5] = 1e4                                      # first NaN wins
        x[2, :] = float("-inf")
        x[3, V - 1] = 3.0                                  # maximum in the scalar tail
        x[4, :] = 2.5                                      # all equal
        x[5, 1] = 1.0
        x[5, 2] = 1.0                                      # tie inside one vector
        idx, val = _check_argmax(x)
        assert idx.tolist() == [0, 77, 0, V - 1, 0, 1]


def test_argmax_unaligned_base_and_leading_dims(cuda):
    gen = torch.Generator(device="cuda").manual_seed(9)
    big = torch.randn(4 * 4099 + 3, generator=gen, device="cuda").bfloat16()
    for off in (1, 3):
        x = big[off:off + 4 * 4099].view(4, 4099)          # rows start at odd element offsets
        _check_argmax(x)
    x3 = torch.randn(2, 3, 515, generator=gen, device="cuda")
    idx, val = ArgmaxRows()(x3)
    assert idx.shape == (2, 3) and torch.equal(idx, x3.argmax(dim=-1))
    only_idx = ArgmaxRows()(x3, with_val=False)
    assert torch.equal(only_idx, idx)
    empty = torch.empty(0, 17, device="cuda")
    idx0, val0 = ArgmaxRows()(empty)
    assert idx0.numel() == 0
    with pytest.raises(QfgError):
        ArgmaxRows()(torch.zeros(2, 8, dtype=torch.int32, device="cuda"))


def test_dequant_fp8_reference_test_case(cuda):
    # the reference's op test: seed 5, K 256, N 128, bit-exact vs (w_fp8.float() * scale).bfloat16()
    gen = torch.Generator(device="cuda").manual_seed(5)
    K, N = 256, 128
    w = (torch.randn(K, N, generator=gen, device="cuda") * 0.05).bfloat16()
    amax = w.float().abs().amax(dim=0).clamp(min=1e-8)
    w_scale = (amax / 448.0).cpu().numpy().astype(np.float32)
    w_fp8 = (w.float() / torch.tensor(w_scale, device="cuda")[None, :]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    out = DequantWeightBf16(N, w_scale=w_scale)(w_fp8)[0]
    ref = (w_fp8.float() * torch.tensor(w_scale, device="cuda")[None, :]).bfloat16()
    assert torch.equal(out, ref)
    q = w_fp8.view(torch.uint8).cpu().numpy()
    assert np.array_equal(bits(out), O.dequant_weight_bf16(1, q, N, 0, w_scale))


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_dequant_slices_and_splits(cuda, mode):
    rng = np.random.default_rng(20 + mode)
    K, N = 96, 512
    arr, _ = U.make_weight(rng, mode, K, N)
    if mode == 2:
        # every scale code at least once, including subnormals, zero, negatives and both NaN codes
        arr[:, N // 2:] = rng.permutation(np.arange(K * (N // 16)) % 256).reshape(K, N // 16).astype(np.uint8)
        arr[0, :4] = [0x88, 0x08, 0x80, 0xF7]
    if mode == 1:
        arr[1, :256] = np.arange(256, dtype=np.uint8)       # every FP8 code
    w = U.dev_weight(arr, mode)
    for n_cols, off, widths, scaled in ((N, 0, None, False), (256, 128, [64, 128, 64], True), (128, 384, [128], True),
                                        (16, 16, None, False)):
        s = rng.uniform(0.25, 4.0, n_cols).astype(np.float32) if scaled and mode != 0 else None
        outs = DequantWeightBf16(n_cols, col_offset=off, widths=widths, w_scale=s)(w)
        torch.cuda.synchronize()
        got = np.concatenate([bits(o) for o in outs], axis=1)
        exp = O.dequant_weight_bf16(mode, arr, n_cols, off, s)
        assert np.array_equal(got, exp), f"mode {mode} slice {off}+{n_cols}"
        assert np.array_equal(exp, C.dequant_bf16(mode, arr, n_cols, off, s))
        assert [o.shape[1] for o in outs] == (widths or [n_cols])


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("K", [1, 3, 6, 97])
def test_dequant_row_counts_off_the_thread_group(cuda, mode, K):
    """A thread converts four consecutive rows of a column chunk: row counts that are not multiples of four
    must not lose the last rows (the kernel guards every row of the group against the row count)."""
    rng = np.random.default_rng(300 + 10 * mode + K)
    N = 192
    arr, _ = U.make_weight(rng, mode, K, N)
    w = U.dev_weight(arr, mode)
    s = rng.uniform(0.25, 4.0, N).astype(np.float32) if mode != 0 else None
    outs = DequantWeightBf16(N, w_scale=s)(w)
    torch.cuda.synchronize()
    assert outs[0].shape == (K, N)
    assert np.array_equal(bits(outs[0]), O.dequant_weight_bf16(mode, arr, N, 0, s))


def test_dequant_errors(cuda):
    with pytest.raises(QfgError):
        DequantWeightBf16(100)                              # not a multiple of 8
    with pytest.raises(QfgError):
        DequantWeightBf16(128, widths=[64, 32])             # widths do not add up
    with pytest.raises(QfgError):
        DequantWeightBf16(128, col_offset=4)
    op = DequantWeightBf16(128, col_offset=64)
    with pytest.raises(QfgError):
        op(torch.zeros((8, 128), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn))  # slice past the row
    with pytest.raises(QfgError):
        op(torch.zeros((8, 256), dtype=torch.float32, device="cuda"))


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("fp8", [False, True])
def test_untile_hc_bf16(cuda, kind, fp8):
    """UntileHcBf16 bit-exact against the oracle; kind 0 also against the construction of the reference's
    own test (tests/test_load.py:404-423)."""
    from qwen38_flash_ops_b200 import UntileHcBf16

    g = torch.Generator(device="cuda").manual_seed(5 + kind)
    cols = 320 if kind == 0 else 10240
    if not fp8:
        src = torch.randint(0, 30000, (160, 20480), dtype=torch.int16, device="cuda", generator=g)
        out = UntileHcBf16(kind)(src.view(torch.bfloat16))
        expect = O.untile_hc_bf16(src.cpu().numpy().view(np.uint16), kind, False)
        assert np.array_equal(bits(out), expect)
        if kind == 0:
            w_orig = torch.randint(0, 30000, (10240, 320), dtype=torch.int16, device="cuda", generator=g)
            tiled = w_orig.view(8, 10, 128, 20, 2, 8).permute(0, 3, 1, 2, 4, 5).contiguous().view(160, 20480)
            assert torch.equal(UntileHcBf16(0)(tiled.view(torch.bfloat16)).view(torch.int16), w_orig)
    else:
        codes = torch.randint(0, 256, (160, 20480), dtype=torch.uint8, device="cuda", generator=g)
        sc = (torch.rand(cols, device="cuda", generator=g) * 0.01 + 1e-4).float()
        out = UntileHcBf16(kind, w_scale=sc.cpu().numpy())(codes.view(torch.float8_e4m3fn))
        expect = O.untile_hc_bf16(codes.cpu().numpy(), kind, True, sc.cpu().numpy())
        got = bits(out)
        nan = (expect & 0x7FFF) > 0x7F80          # E4M3 NaN codes: any NaN pattern is accepted
        assert np.array_equal(got[~nan], expect[~nan]) and np.all((got[nan] & 0x7FFF) > 0x7F80)
        out1 = UntileHcBf16(kind)(codes.view(torch.float8_e4m3fn))     # no scale: factor 1
        expect1 = O.untile_hc_bf16(codes.cpu().numpy(), kind, True, None)
        g1 = bits(out1)
        assert np.array_equal(g1[~nan], expect1[~nan])


def test_untile_hc_rejects_other_shapes(cuda):
    from qwen38_flash_ops_b200 import QfgError, UntileHcBf16

    with pytest.raises(QfgError):
        UntileHcBf16(0)(torch.zeros((160, 20472), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(QfgError):
        UntileHcBf16(2)
