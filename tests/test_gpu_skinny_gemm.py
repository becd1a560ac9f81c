"""GPU parity of SkinnyGemm through the C ABI against the CPU oracle (and, where it was built,
against the reference project's own kernels recompiled for sm_100a).

Tolerance: every output within one BF16 ULP (relative 2^-7) of the FP32-accumulated reference,
plus the accumulation-order term K * 2^-24 * sum|x*w| that any FP32 accumulation is subject to;
the literal 2^-7 criterion is additionally asserted on outputs that do not cancel."""
import numpy as np
import pytest
import torch

from conftest import bits, to_dev
from oracle import cpu as C
from oracle import oracle as O
from qwen38_flash_ops_b200 import QfgError, SkinnyGemm, _lib
from qwen38_flash_ops_b200 import packing as P
from qwen38_flash_ops_b200 import packing_torch as PT

import _util as U

pytestmark = pytest.mark.gpu


def run_case(rng, mode, M, K, seg_widths, with_scale=None, plan=None, force_slow=False, x_bits=None, dense_rows=None):
    """seg_widths: list (per weight) of lists of output widths."""
    seg_outs = [len(w) for w in seg_widths]
    widths = [w for ws in seg_widths for w in ws]
    ns = [sum(ws) for ws in seg_widths]
    x = P.synth_x(rng, M, K) if x_bits is None else x_bits
    stored, scales = [], []
    for n in ns:
        arr, s = U.make_weight(rng, mode, K, n, with_scale)
        stored.append(arr)
        scales.append(s)
    w_scale = None
    if any(s is not None for s in scales):
        w_scale = np.concatenate([s if s is not None else np.ones(n, np.float32) for s, n in zip(scales, ns)])
    op = SkinnyGemm(seg_outs, widths, w_scale=w_scale)
    if plan:
        op.set_option("plan", plan)
    if force_slow:
        op.set_option("force_slow", 1)
    if dense_rows is not None:
        op.set_option("dense_rows", dense_rows)
    outs = op(to_dev(x, "bf16"), *[U.dev_weight(a, mode) for a in stored])
    torch.cuda.synchronize()
    o = 0
    exact = []
    for i, n in enumerate(ns):
        got = np.concatenate([bits(outs[o + j]).reshape(M, -1) for j in range(seg_outs[i])], axis=1)
        s = scales[i] if w_scale is not None and mode != 0 else None
        exact.append(U.check_against_oracle(mode, x, stored[i], n, s, got, K, f"mode{mode} M{M} K{K} seg{i}"))
        o += seg_outs[i]
    return outs, exact


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_small_shapes(cuda, mode, M):
    rng = np.random.default_rng(100 * mode + M)
    run_case(rng, mode, M, 256, [[128]])
    run_case(rng, mode, M, 256, [[64, 64]], with_scale=True)          # the reference test's split (one weight, two outputs)
    run_case(rng, mode, M, 1040, [[192], [64, 128, 64]], with_scale=True)  # two weights, four outputs


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_ragged_shapes(cuda, mode):
    rng = np.random.default_rng(7 + mode)
    n_odd = 192 if mode == 2 else 132          # NVFP4 needs N % 64 == 0; the others N % 4 == 0
    run_case(rng, mode, 2, 250, [[n_odd]])     # K even but not a multiple of 16
    run_case(rng, mode, 3, 34, [[64]])         # K smaller than one stage
    run_case(rng, mode, 1, 2, [[64]])
    if mode != 2:
        run_case(rng, mode, 4, 320, [[4]])     # the reference's 4-column segment
        run_case(rng, mode, 2, 512, [[324 - 4], [4]])
    run_case(rng, mode, 5, 512, [[320]])       # more than four rows in one pass
    run_case(rng, mode, 8, 512, [[320]])
    run_case(rng, mode, 11, 512, [[320]], dense_rows=0)  # two passes of eight and three rows
    if mode == 0:
        run_case(rng, mode, 11, 512, [[320]])  # BF16 weights, more than 8 rows: the library GEMM branch, same tolerance


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("plan", [
    # the register-streaming kernel
    "direct=1,wn=1,wk=16,cluster=1", "direct=1,wn=2,wk=8,cluster=2,ctas=6", "direct=1,wn=4,wk=4,cluster=4",
    "direct=1,wn=8,wk=2,cluster=8", "direct=1,wn=2,wk=2,cluster=1", "direct=1,wn=4,wk=1,cluster=2,ctas=40",
    # the cp.async ring kernel
    "direct=0,wn=1,wk=8,cluster=1", "direct=0,wn=2,wk=4,cluster=2,ctas=6", "direct=0,wn=4,wk=2,cluster=4,stages=3",
    "direct=0,wn=8,wk=1,cluster=8,ks=2,stages=5", "direct=0,wn=2,wk=2,cluster=1,ks=3,stages=2",
    "direct=0,wn=4,wk=1,cluster=2,ctas=40", "direct=1,wn=9,wk=2,cluster=1", "direct=1,wn=3,wk=5,cluster=2",
    # cluster sizes that are not powers of two (the last rank's column share is short)
    "direct=1,wn=2,wk=4,cluster=3", "direct=1,wn=3,wk=2,cluster=6,ctas=18", "direct=0,wn=2,wk=2,cluster=5"])
def test_every_plan_shape(cuda, mode, plan):
    rng = np.random.default_rng(sum(map(ord, plan)) + mode)
    run_case(rng, mode, 3, 2304, [[1280, 256], [512]], with_scale=True, plan=plan)


@pytest.mark.parametrize("stages", [4, 6, 8])
@pytest.mark.parametrize("plan", [
    "wn=1,wk=16,cluster=1", "wn=2,wk=4,cluster=2", "wn=5,wk=3,cluster=1", "wn=1,wk=2,cluster=8",
    "wn=3,wk=4,cluster=1,ctas=7"])
def test_nvfp4_ring_depths_on_misaligned_rows(cuda, stages, plan):
    """Every ring depth of the NVFP4 warp-ring kernel (2, 3 and 4 pairs of k-steps), on weights whose packed
    row pitch is 8 mod 16 (odd rows start half a 16-byte piece off, as in the 151936-column LM head) and on
    one whose pitch is 0 mod 16, with K not a multiple of 16 (zero-filled last k-step) and with odd and even
    numbers of k-steps per warp (a last pair with a single step)."""
    rng = np.random.default_rng(sum(map(ord, plan)) + stages)
    spec = f"direct=1,stages={stages}," + plan
    run_case(rng, 2, 3, 2312, [[640, 384], [896]], plan=spec)
    run_case(rng, 2, 8, 1000, [[1280], [128, 128]], plan=spec)
    run_case(rng, 2, 2, 16 * 7, [[384]], plan=spec)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_row_independence_and_determinism(cuda, mode):
    """Row r of an M-row call is bit-identical to the one-row call on that row, and a repeated
    call is bit-identical to the first."""
    rng = np.random.default_rng(40 + mode)
    K, N = 1536, 640
    arr, s = U.make_weight(rng, mode, K, N, True)
    x = P.synth_x(rng, 8, K)
    # make the rows differ in scale by orders of magnitude (row-wise power-of-two prescale)
    xf = O.bf16_to_f32(x)
    xf *= np.array([1, 1e-3, 300, 1, 2e4, 1e-6, 1, 1], np.float32)[:, None]
    x = P.f32_to_bf16_bits(xf)
    op = SkinnyGemm([1], [N], w_scale=s if mode != 0 else None)
    w = U.dev_weight(arr, mode)
    full = bits(op(to_dev(x, "bf16"), w)[0])
    again = bits(op(to_dev(x, "bf16"), w)[0])
    assert np.array_equal(full, again)
    for M in (1, 2, 4):
        part = bits(op(to_dev(x[:M], "bf16"), w)[0])
        assert np.array_equal(part, full[:M]), f"M={M} differs from the 8-row call"
    for r in range(8):
        one = bits(op(to_dev(x[r:r + 1], "bf16"), w)[0])
        assert np.array_equal(one[0], full[r]), f"row {r} differs from its one-row call"
    U.check_against_oracle(mode, x, arr, N, s if mode != 0 else None, full, K, "row-scaled")


@pytest.mark.parametrize("mode", [1, 2])
def test_wide_dynamic_range_takes_bf16_path(cuda, mode):
    """x whose K slice spans more than 2^28 is not exactly representable in FP16 after the
    power-of-two prescale; the CTA then runs the BF16 MMA on exact BF16 operands.  Both paths
    must satisfy the tolerance; on ordinary inputs they must agree bit for bit."""
    rng = np.random.default_rng(50 + mode)
    K, N = 1024, 384
    arr, s = U.make_weight(rng, mode, K, N, True)
    x = O.bf16_to_f32(P.synth_x(rng, 2, K))
    x[0, 5] = 3e30
    x[0, 6] = 1e-30
    x[1, 100] = np.float32(2.0 ** -120)
    xb = P.f32_to_bf16_bits(x)
    op = SkinnyGemm([1], [N], w_scale=s)
    w = U.dev_weight(arr, mode)
    got = bits(op(to_dev(xb, "bf16"), w)[0])
    U.check_against_oracle(mode, xb, arr, N, s, got, K, "wide range")
    # inf / nan inputs propagate like IEEE arithmetic
    x2 = O.bf16_to_f32(P.synth_x(rng, 2, K))
    x2[0, 3] = np.inf
    x2[1, 4] = np.nan
    xb2 = P.f32_to_bf16_bits(x2)
    got2 = O.bf16_to_f32(bits(op(to_dev(xb2, "bf16"), w)[0]))
    ref2, _, _ = C.skinny_gemm(mode, xb2, arr, N, s)
    ref2 = O.bf16_to_f32(ref2)
    assert np.array_equal(np.isnan(got2), np.isnan(ref2))
    assert np.array_equal(np.isinf(got2), np.isinf(ref2))
    # ordinary inputs: forced BF16 path == FP16 path
    xo = P.synth_x(rng, 4, K)
    fast = bits(op(to_dev(xo, "bf16"), w)[0])
    op.set_option("force_slow", 1)
    slow = bits(op(to_dev(xo, "bf16"), w)[0])
    U.check_against_oracle(mode, xo, arr, N, s, slow, K, "forced bf16 path")
    assert np.array_equal(fast, slow), f"{np.count_nonzero(fast != slow)} outputs differ between the two MMA paths"


def test_guard_bands_untouched(cuda):
    rng = np.random.default_rng(60)
    K, widths = 512, [64, 192, 64]
    for mode in (0, 1, 2):
        arr, s = U.make_weight(rng, mode, K, sum(widths), True)
        for M in (1, 4, 7):
            x = P.synth_x(rng, M, K)
            pad = 64
            bufs = [torch.full((M * w + 2 * pad,), -12851, dtype=torch.int16, device="cuda") for w in widths]  # 0xCDCD
            outs = [b[pad:pad + M * w].view(torch.bfloat16).view(M, w) for b, w in zip(bufs, widths)]
            op = SkinnyGemm([3], widths, w_scale=s if mode != 0 else None)
            op(to_dev(x, "bf16"), U.dev_weight(arr, mode), out=outs)
            torch.cuda.synchronize()
            for b, w in zip(bufs, widths):
                h = b.cpu().numpy()
                assert np.all(h[:pad] == -12851) and np.all(h[pad + M * w:] == -12851)
            got = np.concatenate([bits(o) for o in outs], axis=1)
            U.check_against_oracle(mode, x, arr, sum(widths), s if mode != 0 else None, got, K, "guard")


@pytest.mark.parametrize("trigger,pdl_wait", [(0, 0), (1, 0), (2, 0), (1, 1), (2, 1)])
def test_cuda_graph_capture_and_pdl(cuda, trigger, pdl_wait):
    """The compute call is capturable; replaying the graph gives the eager result.  With the
    PDL trigger set, a chain of dependent calls (each consuming the previous output as x) stays
    correct when the kernels are launched with programmatic stream serialisation."""
    rng = np.random.default_rng(70)
    K = N = 512
    arr, _ = U.make_weight(rng, 2, K, N)
    w = U.dev_weight(arr, 2)
    x0 = to_dev(P.synth_x(rng, 4, K), "bf16")
    op = SkinnyGemm([1], [N], trigger=trigger)
    op.set_option("pdl_wait", pdl_wait)
    plain = SkinnyGemm([1], [N])

    def chain(o, x):
        y1 = o(x, w)[0]
        y2 = o(y1, w)[0]
        return o(y2, w)[0]

    expect = bits(chain(plain, x0))
    eager = bits(chain(op, x0))
    assert np.array_equal(eager, expect)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        chain(op, x0)  # warm-up on the capture stream
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            y = chain(op, x0)
        for _ in range(3):
            g.replay()
    torch.cuda.synchronize()
    assert np.array_equal(bits(y), expect)


def test_argument_errors(cuda):
    rng = np.random.default_rng(80)
    K, N = 256, 128
    x = to_dev(P.synth_x(rng, 2, K), "bf16")
    wb = U.dev_weight(P.f32_to_bf16_bits(P.synth_weight(rng, K, N)), 0)
    op = SkinnyGemm([1], [N])
    with pytest.raises(QfgError) as e:
        op(x, wb, wb)                                   # input count
    assert e.value.code == _lib.QFG_INVALID_ARGUMENT
    with pytest.raises(QfgError):
        op(x[:, :254].contiguous(), wb)                 # weight rows != K
    with pytest.raises(QfgError):
        SkinnyGemm([1], [N - 4])(x, wb)                 # widths do not add up to N
    with pytest.raises(QfgError):
        SkinnyGemm([1], [130])(x, U.dev_weight(np.zeros((K, 130), np.uint16), 0))   # N % 4
    with pytest.raises(QfgError):
        SkinnyGemm([1], [N])(x, torch.zeros((K, N * 9 // 16 + 1), dtype=torch.uint8, device="cuda"))
    with pytest.raises(QfgError):
        SkinnyGemm([1], [48])(x, torch.zeros((K, 27), dtype=torch.uint8, device="cuda"))  # NVFP4 N % 64
    with pytest.raises(QfgError):
        SkinnyGemm([1], [N])(x, torch.zeros((K, N), dtype=torch.float32, device="cuda"))   # element type
    with pytest.raises(QfgError):
        SkinnyGemm([1, 1], [N, N])(x, wb, U.dev_weight(np.zeros((K, N), np.uint8), 1))     # mixed types
    xo = to_dev(P.synth_x(rng, 2, 255), "bf16")
    with pytest.raises(QfgError):
        SkinnyGemm([1], [N])(xo, U.dev_weight(np.zeros((255, N), np.uint16), 0))           # odd K
    # after all those refusals the op still works
    y = op(x, wb)[0]
    torch.cuda.synchronize()
    assert y.shape == (2, N)


CONFIGS = {
    # name: (mode, M, K, seg widths)
    "C1_bf16": (0, 1, 5120, [[5120]]),
    "C2_fp8_qkv": (1, 2, 5120, [[8192], [1024], [1024]]),
    "C3_nvfp4_gate_up": (2, 1, 5120, [[17408], [17408]]),
    "C4_nvfp4_down": (2, 4, 17408, [[5120]]),
}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_baseline_configs_full_size(cuda, name):
    """The benchmark configurations at full size: weights generated and packed on the GPU, the C
    oracle (FP64 accumulation, all host cores) as the checker, plus the reference kernels."""
    mode, M, K, seg_widths = CONFIGS[name]
    gen = torch.Generator(device="cuda").manual_seed(0x5EED0000 + len(name))
    rng = np.random.default_rng(0x5EED0000 + len(name))
    x = P.synth_x(rng, M, K)
    xd = to_dev(x, "bf16")
    ws, scales, ns = [], [], []
    for wsz in seg_widths:
        n = sum(wsz)
        w = torch.randn(K, n, generator=gen, device="cuda") * 0.02
        if mode == 0:
            ws.append(w.bfloat16())
            scales.append(None)
        elif mode == 1:
            q, s = PT.quantize_fp8_per_column_torch(w)
            ws.append(q)
            scales.append(s)
        else:
            ws.append(PT.pack_nvfp4_torch(w))
            scales.append(None)
        ns.append(n)
        del w
    w_scale = torch.cat(scales).cpu().numpy() if mode == 1 else None
    seg_outs = [len(w) for w in seg_widths]
    widths = [w for wsz in seg_widths for w in wsz]
    op = SkinnyGemm(seg_outs, widths, w_scale=w_scale, trigger=2 if name.startswith("C4") else 0)
    outs = op(xd, *ws)
    torch.cuda.synchronize()
    for i, n in enumerate(ns):
        host = ws[i].view(torch.uint8).cpu().numpy() if mode != 0 else bits(ws[i])
        s = scales[i].cpu().numpy() if scales[i] is not None else None
        U.check_against_oracle(mode, x, host, n, s, bits(outs[i]), K, f"{name} seg{i}")
    if U.ref_lib() is not None:
        r = U.ref_skinny_gemm(xd, ws, [mode] * len(ws), ns, scales, seg_outs, widths)
        torch.cuda.synchronize()
        for a, b in zip(outs, r):
            d = np.abs(bits(a).astype(np.int32) - bits(b).astype(np.int32))
            assert np.mean(d <= 1) > 0.999, f"{name}: differs from the reference kernel by more than one BF16 ULP"
            # observed: 0.9995 - 0.99995 of the outputs bit-identical (different FP32 summation orders)
            assert np.mean(d == 0) > 0.999, f"{name}: only {np.mean(d == 0):.5f} of the outputs equal the reference kernel's"


def test_linearity_at_full_size(cuda):
    """Size-independent property at a benchmark size: y(x with one element doubled) - y(x) equals
    that element times the weight row, exactly representable here, within the output rounding."""
    K, N = 5120, 17408
    gen = torch.Generator(device="cuda").manual_seed(99)
    pk = PT.pack_nvfp4_torch(torch.randn(K, N, generator=gen, device="cuda") * 0.02)
    op = SkinnyGemm([1], [N])
    x = torch.zeros(2, K, dtype=torch.bfloat16, device="cuda")
    x[0, 1234] = 1.0
    x[1, 4321] = -2.0
    y = op(x, pk)[0].float().cpu().numpy()
    host = pk.cpu().numpy()
    rows = O.decode_weights_exact(2, host[[1234, 4321]], N)
    assert np.array_equal(y[0], rows[0])      # one-hot x reads back the dequantised row exactly
    assert np.array_equal(y[1], -2.0 * rows[1])


@pytest.mark.parametrize("plan", [
    "wn=4,wk=2,cluster=1", "wn=4,wk=3,cluster=2", "wn=8,wk=2,cluster=1,stages=3", "wn=4,wk=1,cluster=4,stages=6",
    "wn=4,wk=3,cluster=1,ctas=5"])
def test_nvfp4_tensor_memory_kernel(cuda, plan):
    """The tcgen05 variant of the NVFP4 kernel (A fragments in tensor memory, one issuing warp, mma.sync
    warps for the columns past the warpgroups): aligned and 8-mod-16 row pitches, K not a multiple
    of 16, 1 to 8 rows, tiles that need the extra columns and tiles that leave warps empty."""
    rng = np.random.default_rng(sum(map(ord, plan)))
    spec = "direct=1,tc=1,wide=1," + plan
    run_case(rng, 2, 3, 2312, [[640, 384], [896]], plan=spec)
    run_case(rng, 2, 8, 1000, [[1280], [128, 128]], plan=spec)
    run_case(rng, 2, 1, 2048, [[4096 + 128]], with_scale=True, plan=spec)


def test_nvfp4_tensor_memory_kernel_matches_direct_kernel_on_wide_range(cuda):
    """x with a dynamic range that forces the BF16 operand path: the tcgen05 kernel (BF16 kind) and the
    mma.sync kernel see the same exact operands and must both satisfy the oracle."""
    rng = np.random.default_rng(4242)
    K, N = 1024, 1024
    x = P.synth_x(rng, 4, K)
    xf = O.bf16_to_f32(x)
    xf[:, ::7] *= 2.0 ** 20
    xf[:, 1::7] *= 2.0 ** -20
    x = P.f32_to_bf16_bits(xf)
    run_case(rng, 2, 4, K, [[N]], plan="direct=1,tc=1,wide=1,wn=4,wk=2,cluster=1", x_bits=x)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("plan", [
    "direct=2,wn=1,wk=16,cluster=1", "direct=2,wn=2,wk=8,cluster=2,ctas=6", "direct=2,wn=4,wk=4,cluster=4",
    "direct=2,wn=8,wk=2,cluster=8", "direct=2,wn=2,wk=2,cluster=1", "direct=2,wn=4,wk=1,cluster=2,ctas=40"])
def test_register_streaming_kernel(cuda, mode, plan):
    """The BF16 / FP8 variant that loads weights straight into registers (no shared-memory ring)."""
    rng = np.random.default_rng(sum(map(ord, plan)) + mode)
    run_case(rng, mode, 3, 2304, [[1280, 256], [512]], with_scale=True, plan=plan)
    run_case(rng, mode, 8, 1000, [[640], [128, 128]], with_scale=True, plan=plan)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_many_rows_take_the_dense_branch(cuda, mode):
    """Prefill-shaped calls (more rows than the `dense_rows` option; by default 8 / 8 / 16 for BF16 / FP8 / NVFP4) dequantise the weights to
    BF16 with w_scale folded in and run a library GEMM, as the reference does for M > 8 (fused_gemm.cu:365-428).
    The accumulation order of that GEMM is not pinned, so the check is the tolerance against the exact sum over
    the BF16-rounded weights, and agreement with the streaming passes within the rounding of those weights."""
    rng = np.random.default_rng(900 + mode)
    M, K = 80, 1024
    seg_widths = [[256], [128, 384]]
    seg_outs = [len(w) for w in seg_widths]
    widths = [w for ws in seg_widths for w in ws]
    ns = [sum(ws) for ws in seg_widths]
    x = P.synth_x(rng, M, K)
    stored, scales = zip(*[U.make_weight(rng, mode, K, n, True) for n in ns])
    quantised = mode != 0
    w_scale = np.concatenate(scales) if quantised else None
    dense = SkinnyGemm(seg_outs, widths, w_scale=w_scale)
    passes = SkinnyGemm(seg_outs, widths, w_scale=w_scale)
    passes.set_option("dense_rows", 0)
    xd = to_dev(x, "bf16")
    wd = [U.dev_weight(a, mode) for a in stored]
    out_dense = dense(xd, *wd)
    out_passes = passes(xd, *wd)
    # rows at or below the threshold keep the streaming kernels: bit-identical with the branch switched off
    small = {0: 8, 1: 8, 2: 16}[mode]
    out_small = dense(xd[:small], *wd)
    torch.cuda.synchronize()
    o = 0
    for i, n in enumerate(ns):
        cat = lambda outs, rows: np.concatenate([bits(outs[o + j]).reshape(rows, -1) for j in range(seg_outs[i])], axis=1)
        got, ref_passes = cat(out_dense, M), cat(out_passes, M)
        assert np.array_equal(cat(out_small, small), ref_passes[:small])
        w_bf16 = O.dequant_weight_bf16(mode, stored[i], n, 0, scales[i] if quantised else None)
        _, sums, mags = C.skinny_gemm(0, x, w_bf16, n, None)
        ok = O.gemm_within_tolerance(got, sums, mags, K)
        assert ok.all(), f"mode {mode} weight {i}: {np.count_nonzero(~ok)} outputs outside tolerance"
        a, b = O.bf16_to_f32(got).astype(np.float64), O.bf16_to_f32(ref_passes).astype(np.float64)
        # the two branches round the scaled weights at different points: 2^-9 relative per weight
        assert (np.abs(a - b) <= 2.0 ** -7 * np.abs(b) + 2.0 ** -8 * mags + 1e-30).all()
        U.check_against_oracle(mode, x, stored[i], n, scales[i] if quantised else None, ref_passes, K, "passes")
        o += seg_outs[i]


def test_dense_branch_tiles_wide_outputs_and_skips_odd_widths(cuda):
    """An output wider than one dequantisation tile (16384 columns) is produced tile by tile; widths that are
    not multiples of eight stay on the streaming kernels at any row count."""
    rng = np.random.default_rng(77)
    M, K, n = 40, 128, 16384 + 4096
    x = P.synth_x(rng, M, K)
    w, s = U.make_weight(rng, 2, K, n, True)
    op = SkinnyGemm([1], [n], w_scale=s)
    out = op(to_dev(x, "bf16"), U.dev_weight(w, 2))
    torch.cuda.synchronize()
    w_bf16 = O.dequant_weight_bf16(2, w, n, 0, s)
    _, sums, mags = C.skinny_gemm(0, x, w_bf16, n, None)
    assert O.gemm_within_tolerance(bits(out[0]).reshape(M, n), sums, mags, K).all()
    # 100 columns: not a multiple of eight -> the streaming kernels at M = 40, row by row as for one row
    w2, _ = U.make_weight(rng, 0, K, 100)
    op2 = SkinnyGemm([1], [100])
    out2 = op2(to_dev(x, "bf16"), U.dev_weight(w2, 0))
    torch.cuda.synchronize()
    U.check_against_oracle(0, x, w2, 100, None, bits(out2[0]).reshape(M, 100), K, "odd width")
    one = op2(to_dev(x[17:18], "bf16"), U.dev_weight(w2, 0))
    torch.cuda.synchronize()
    assert np.array_equal(bits(one[0]).reshape(-1), bits(out2[0]).reshape(M, 100)[17])


def test_trigger_attribute_and_its_environment_override(cuda, monkeypatch):
    """SKINNY_TRIGGER_FORCE=<n> replaces a non-zero `trigger` attribute when the node is created and leaves a
    zero attribute alone (fused_gemm.cu:105-113)."""
    w = to_dev(np.zeros((64, 128), np.uint16), "bf16")

    def resolved(trigger):
        fields = dict(item.split("=") for item in SkinnyGemm([1], [128], trigger=trigger).describe(64, w).split(","))
        return int(fields["trigger"])

    monkeypatch.delenv("SKINNY_TRIGGER_FORCE", raising=False)
    assert [resolved(t) for t in (0, 1, 2)] == [0, 1, 2]
    monkeypatch.setenv("SKINNY_TRIGGER_FORCE", "1")
    assert [resolved(t) for t in (0, 1, 2)] == [0, 1, 1]
    monkeypatch.setenv("SKINNY_TRIGGER_FORCE", "0")
    assert [resolved(t) for t in (0, 2)] == [0, 0]
