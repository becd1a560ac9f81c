"""GPU parity of the fused LM head (SkinnyGemm + ArgmaxRows in one kernel) and of its N-sharded
form emulated on one GPU: shards run one after the other, keys are combined like the all-gathered
payload would be."""
import numpy as np
import pytest
import torch

from conftest import bits, to_dev
from oracle import cpu as C
from oracle import oracle as O
from qwen38_flash_ops_b200 import ArgmaxRows, LmHeadArgmax, SkinnyGemm, lmhead_combine
from qwen38_flash_ops_b200 import packing as P
from qwen38_flash_ops_b200 import packing_torch as PT

import _util as U

pytestmark = pytest.mark.gpu


def _oracle_near_tie_ok(idx_got, sums, logits_bits_oracle, idx_oracle):
    """An index that differs from the oracle's is acceptable only if the two candidates' oracle
    logits are within one BF16 ULP of each other (the kernel's FP32 sum may round the other way)."""
    bad = 0
    for r in range(len(idx_got)):
        if idx_got[r] == idx_oracle[r]:
            continue
        a = int(logits_bits_oracle[r, idx_got[r]])
        b = int(logits_bits_oracle[r, idx_oracle[r]])
        if abs(a - b) > 1:
            bad += 1
    return bad


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("M", [1, 2, 4, 8])
def test_fused_equals_unfused_chain(cuda, mode, M):
    rng = np.random.default_rng(300 + 10 * mode + M)
    K, N = 768, 4096 + 64
    arr, s = U.make_weight(rng, mode, K, N, True)
    x = P.synth_x(rng, M, K)
    xd, w = to_dev(x, "bf16"), U.dev_weight(arr, mode)
    scale = s if mode != 0 else None
    logits = SkinnyGemm([1], [N], w_scale=scale)(xd, w)[0]
    eidx, eval_ = ArgmaxRows()(logits)
    head = LmHeadArgmax(w_scale=scale)
    for rep in range(3):   # the workspace must come back clean after every call
        idx, val, key, lg = head(xd, w, N, logits=True)
        torch.cuda.synchronize()
        assert torch.equal(lg, logits)
        assert torch.equal(idx, eidx), f"rep {rep}"
        assert torch.equal(val, eval_)
        assert int(head.workspace.view(torch.int64).abs().sum().item()) == 0
    idx2, val2, key2 = head(xd, w, N, col_offset=1000)
    assert torch.equal(idx2, eidx + 1000)
    # against the FP64 oracle, allowing only near-ties
    obits, sums, mags = C.skinny_gemm(mode, x, arr, N, scale)
    oidx, oval = C.argmax_rows(0, obits)
    assert _oracle_near_tie_ok(idx.cpu().numpy(), sums, obits, oidx) == 0


def test_planted_ties_and_nan(cuda):
    rng = np.random.default_rng(77)
    K, N = 256, 2048
    w = np.zeros((K, N), np.float32)
    w[0, 300] = w[0, 1700] = w[0, 40] = 0.5            # three equal maxima: lowest index wins
    wb = P.f32_to_bf16_bits(w)
    x = np.zeros((2, K), np.float32)
    x[0, 0] = 2.0
    x[1, 0] = -1.0                                     # row 1: all logits <= 0, the maximum 0 first at column 0
    xb = P.f32_to_bf16_bits(x)
    head = LmHeadArgmax()
    idx, val, key = head(to_dev(xb, "bf16"), U.dev_weight(wb, 0), N)
    assert idx.tolist() == [40, 0] and val.tolist() == [1.0, 0.0]
    wn = w.copy()
    wn[0, 900] = np.nan
    wn[0, 100] = np.nan
    idx, val, key = head(to_dev(xb, "bf16"), U.dev_weight(P.f32_to_bf16_bits(wn), 0), N)
    assert idx.tolist() == [100, 100] and bool(torch.isnan(val).all())


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_emulation_matches_single(cuda, world):
    rng = np.random.default_rng(400 + world)
    K, N, M = 512, 128 * 37, 4
    pk = P.pack_nvfp4(P.synth_weight(rng, K, N))
    x = P.synth_x(rng, M, K)
    xd = to_dev(x, "bf16")
    head = LmHeadArgmax()
    idx1, val1, key1 = head(xd, to_dev(pk, "u8"), N)
    keys = torch.empty((world, M), dtype=torch.int64, device="cuda")
    for r, (c0, c1) in enumerate(P.shard_columns(N, world)):
        shard = to_dev(P.nvfp4_column_slice(pk, N, c0, c1), "u8")
        _, _, k = head(xd, shard, c1 - c0, col_offset=c0)
        keys[r] = k
    idx, val = lmhead_combine(keys, world, M)
    torch.cuda.synchronize()
    assert torch.equal(idx, idx1) and torch.equal(val, val1)


@pytest.mark.parametrize("M", [1, 2, 4])
def test_lmhead_full_vocabulary(cuda, M):
    """The benchmark LM head (K 5120, vocabulary 151936, NVFP4) at full size against the C oracle."""
    K, N = 5120, 151936
    gen = torch.Generator(device="cuda").manual_seed(0x5EED0005)
    pk = torch.empty((K, N * 9 // 16), dtype=torch.uint8, device="cuda")
    for c0 in range(0, N, 18992 * 2):                       # pack in column blocks to bound memory
        c1 = min(N, c0 + 18992 * 2)
        blk = PT.pack_nvfp4_torch(torch.randn(K, c1 - c0, generator=gen, device="cuda") * 0.02)
        pk[:, c0 // 2:c1 // 2] = blk[:, :(c1 - c0) // 2]
        pk[:, N // 2 + c0 // 16:N // 2 + c1 // 16] = blk[:, (c1 - c0) // 2:]
    rng = np.random.default_rng(0x5EED0005)
    x = P.synth_x(rng, M, K)
    xd = to_dev(x, "bf16")
    head = LmHeadArgmax()
    idx, val, key, lg = head(xd, pk, N, logits=True)
    logits = SkinnyGemm([1], [N])(xd, pk)[0]
    eidx, eval_ = ArgmaxRows()(lg)
    torch.cuda.synchronize()
    # the argmax is exact on the logits the fused kernel itself produced ...
    assert torch.equal(idx, eidx) and torch.equal(val, eval_)
    # ... which are the plain kernel's logits, except that the 3 column groups the 148 CTAs share
    # (151936 = 148 x 8 x 128 + 3 x 128) are summed over K in another fixed order: at most one BF16 ULP
    shared = 3 * 128
    assert torch.equal(lg[:, :N - shared], logits[:, :N - shared])
    d = (bits(lg[:, N - shared:]).astype(np.int32) - bits(logits[:, N - shared:]).astype(np.int32))
    assert np.abs(d).max() <= 1 and np.mean(d == 0) > 0.95
    host = pk.cpu().numpy()
    U.check_against_oracle(2, x, host, N, None, bits(logits), K, "lm head")
    obits, sums, mags = C.skinny_gemm(2, x, host, N, None)
    oidx, _ = C.argmax_rows(0, obits)
    assert _oracle_near_tie_ok(idx.cpu().numpy(), sums, obits, oidx) == 0
    if U.ref_lib() is not None:
        r = U.ref_skinny_gemm(xd, [pk], [2], [N], [None], [1], [N])[0]
        ridx, rval = U.ref_argmax_rows(r)
        torch.cuda.synchronize()
        d = np.abs(bits(r).astype(np.int32) - bits(logits).astype(np.int32))
        assert np.mean(d <= 1) > 0.999
        assert np.mean(d == 0) > 0.999  # observed: 0.9998 of the logits bit-identical to the reference kernel's
        assert _oracle_near_tie_ok(ridx.cpu().numpy(), sums, obits, oidx) == 0


def test_host_buffer_head_matches_device_step(cuda):
    """HostLmHead (pinned host x in, idx / val out, one captured graph) returns what the
    device-resident step returns, call after call, for changing inputs."""
    from qwen38_flash_ops_b200.lmhead_shard import HostLmHead, ShardedLmHead

    rng = np.random.default_rng(77)
    K, N, M = 1024, 1280, 3
    arr, _ = U.make_weight(rng, 2, K, N, False)
    w = U.dev_weight(arr, 2)
    head = ShardedLmHead(w, N, 0)
    host = HostLmHead(head, M, K)
    for trial in range(3):
        x = P.synth_x(rng, M, K)
        xd = to_dev(x, "bf16")
        idx, val = head.step(xd)
        ih, vh = host(xd.cpu())
        assert torch.equal(ih, idx.cpu()) and torch.equal(vh, val.cpu()), f"trial {trial}"


@pytest.mark.parametrize("M", [1, 4, 8])
@pytest.mark.parametrize("tail", [1, 3])
def test_lmhead_shared_tail_columns(cuda, M, tail):
    """Column groups left over by the CTA count are computed by all CTAs together (each a share of the K
    range, partial sums added by the last CTA).  The fused result must still equal
    ArgmaxRows(SkinnyGemm(x)) of the plain kernel bit for bit, logits of the tail columns included,
    also when the best column lies in the tail."""
    rng = np.random.default_rng(900 + M + 10 * tail)
    K = 1000                                   # 63 k-steps, the last one partial
    ctas, per = 5, 2
    N = (ctas * per + tail) * 128
    arr, _ = U.make_weight(rng, 2, K, N, False)
    w = U.dev_weight(arr, 2)
    x = P.synth_x(rng, M, K)
    xd = to_dev(x, "bf16")
    plain = SkinnyGemm([1], [N])
    plain.set_option("plan", "direct=1,wide=1,wn=3,wk=2,cluster=1,ctas=5")
    logits = plain(xd, w)[0]
    eidx, eval_ = ArgmaxRows()(logits)
    head = LmHeadArgmax()
    head.set_option("plan", f"direct=1,wide=1,wn=3,wk=2,cluster=1,ctas={ctas},tail={tail}")
    for _ in range(2):                          # twice: the workspace must come back clean
        idx, val, key, lg = head(xd, w, N, logits=True)
        torch.cuda.synchronize()
        shared = tail * 128
        assert torch.equal(lg[:, :N - shared], logits[:, :N - shared])
        d = bits(lg[:, N - shared:]).astype(np.int32) - bits(logits[:, N - shared:]).astype(np.int32)
        assert np.abs(d).max() <= 1 and np.mean(d == 0) > 0.9, "shared columns: another summation order, one ULP at most"
        eidx, eval_ = ArgmaxRows()(lg)
        assert torch.equal(idx, eidx) and torch.equal(val, eval_)
    U.check_against_oracle(2, x, arr, N, None, bits(lg), K, "lm head with shared tail")
    # the winner must be found when it lies in the shared columns: repeat on a weight whose other columns are zeroed
    arr2 = arr.copy()
    arr2[:, :(N - tail * 128) // 2] = 0         # nibbles of the non-shared columns -> all logits there are +0
    w2 = U.dev_weight(arr2, 2)
    idx2, val2, _, lg2 = head(xd, w2, N, logits=True)
    eidx2, eval2 = ArgmaxRows()(lg2)
    torch.cuda.synchronize()
    assert torch.equal(idx2, eidx2) and torch.equal(val2, eval2)
    assert bool(torch.all(idx2 >= N - tail * 128) | torch.all(val2 <= 0))
