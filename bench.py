#!/usr/bin/env python3
"""Benchmark of the decode weight-streaming path (SkinnyGemm / fused LM head) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows M]

Headline workload: the NVFP4 LM head (K 5120, vocabulary 151936, `UINT8 [5120, 85464]`, 437.6 MB
of packed weights - larger than L2, so every step streams from HBM) fused with ArgmaxRows.  One
step is one call on one batch of M rows; with N > 1 GPUs the vocabulary is split by columns
(128-column granules), every rank runs the fused kernel on its shard and the ranks exchange their
per-row (max, index) keys - inside the fused kernel, whose last CTA stores them into every rank's
peer-mapped buffer and folds what arrives (the timed path), with the NCCL all-gather + fold kernel
timed beside it (`exchange_alt`).  Total work is fixed, so scaling is strong.  The metric is weight
bytes per second over all GPUs.  Rank 0 prints one JSON line.

`--impl reference` times the CPU restatement of the unfused chain the op replaces (dequantise ->
MatMul with FP32 accumulation -> ArgMax) on all host cores over the whole head, once per step; the
reference project has no CPU implementation of its own, and ONNX Runtime is not installed here.
Where the reference's CUDA kernels were compiled for sm_100a (oracle/_ref) their time on the same
workload is reported beside it.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "nvfp4_skinny_gemm_weight_stream"
UNIT = "TB/s"
HEAD = "C5_nvfp4_lmhead_5120x151936"


# DRAM sectors per launch of the fused LM-head kernel, from an ncu capture of this workload:
# (439.54 MB read + 4.58 MB written) / 437.58 MB of packed weights
NCU_DRAM_BYTES_PER_WEIGHT_BYTE = 1.0150


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("hbm_gbs", 6459.6), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and clock-event reasons through NVML (read-only) while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.sm, self.reasons = [], set()
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.thread = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.sm.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.003)

    def stop(self):
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.sm)}


def time_region(torch, fn, steps, warmup, dist=None):
    """W warm-up calls, then exactly `steps` calls bracketed by barrier + synchronize; device time
    from CUDA events on the launching stream; max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def time_graph_rotation(torch, make_call, n_buffers, reps=20, warmup=3):
    """Per-call device time of a short kernel: a CUDA graph holding one call per weight copy
    (copies total more than 16x L2, so every call streams from HBM), replayed `reps` times."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(n_buffers):
            make_call(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(n_buffers):
                make_call(i)
        for _ in range(warmup):
            g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1000.0 / n_buffers)
    return statistics.median(times), min(times)


def bench_small_configs(torch, quick=False):
    """Configs C1-C4 (50-100 MB, L2-sized): device-timed us/call under buffer rotation, weight GB/s."""
    from qwen38_flash_ops_b200 import SkinnyGemm
    from qwen38_flash_ops_b200 import workloads as W

    peak, _ = peaks()
    out = {}
    for name, wl in W.CONFIGS.items():
        if wl.fused_argmax:
            continue
        copies = max(2, min(48, -(-(2 << 30) // wl.weight_bytes)))
        if quick:
            copies = min(copies, 8)
        sets, scales = [], None
        for c in range(copies):
            ws = []
            sc = []
            for i, n in enumerate(wl.ns):
                w, s = W.make_weight(wl.mode, wl.k, n, seed=1000 * c + i)
                ws.append(w)
                sc.append(s)
            sets.append(ws)
            if c == 0 and wl.mode == W.MODE_FP8:
                scales = torch.cat(sc).cpu().numpy()
        seg_outs = [len(w) for w in wl.seg_widths]
        widths = [w for ws_ in wl.seg_widths for w in ws_]
        res = {"weight_bytes": wl.weight_bytes, "copies": copies}
        for m in sorted({1, 2, 4, wl.m}):
            x = W.make_x(m, wl.k, seed=7)
            outs = [torch.empty((m, w), dtype=torch.bfloat16, device="cuda") for w in widths]
            for label, pdl in (("", 0), ("_pdl", 1)):
                op = SkinnyGemm(seg_outs, widths, w_scale=scales, trigger=(wl.trigger or 2) if pdl else wl.trigger)
                op.set_option("pdl_wait", pdl)
                med, best = time_graph_rotation(torch, lambda i: op(x, *sets[i], out=outs), copies)
                res[f"M{m}{label}"] = {"us": round(med, 3), "us_best": round(best, 3),
                                       "GBps": round(wl.weight_bytes / med / 1e3, 1),
                                       "frac_of_measured_hbm": round(wl.weight_bytes / med / 1e3 / peak, 4),
                                       "frac_of_8TBps": round(wl.weight_bytes / med / 1e3 / 8000.0, 4)}
        ref = _ref_util()
        if ref is not None:
            # the reference project's own kernels (generic launch configuration) under the same rotation
            x = W.make_x(wl.m, wl.k, seed=7)
            sc_dev = [None] * len(wl.ns)
            if scales is not None:
                offs = [0]
                for n in wl.ns:
                    offs.append(offs[-1] + n)
                full = torch.tensor(scales, dtype=torch.float32, device="cuda")
                sc_dev = [full[offs[i]:offs[i + 1]].contiguous() for i in range(len(wl.ns))]
            modes = [wl.mode] * len(wl.ns)
            med, best = time_graph_rotation(
                torch, lambda i: ref.ref_skinny_gemm(x, sets[i], modes, list(wl.ns), sc_dev, seg_outs, widths), copies)
            res["reference_kernel_sm100a"] = {"rows": wl.m, "us": round(med, 3), "us_best": round(best, 3),
                                              "GBps": round(wl.weight_bytes / med / 1e3, 1)}
        res["plan"] = SkinnyGemm(seg_outs, widths, w_scale=scales).describe(wl.k, *sets[0])
        out[name] = res
        del sets
        torch.cuda.empty_cache()
    return out


def bench_model_shapes(torch):
    """Shapes outside the benchmark's own five, taken from the launch table of the reference operator
    (src/fused_gemm/fused_gemm.cu:132-156: the projections of a K = 2560 model) plus two NVFP4 ones: none of
    them is in this build's tuned table, so the scoring rule of the planner picks their launch shapes.  One row,
    device time per call under buffer rotation, the reference's kernel (generic configuration) beside it."""
    from qwen38_flash_ops_b200 import SkinnyGemm
    from qwen38_flash_ops_b200 import workloads as W

    ref = _ref_util()
    shapes = [(W.MODE_BF16, 2560, 16480), (W.MODE_BF16, 2560, 12800), (W.MODE_BF16, 2560, 1792), (W.MODE_BF16, 6144, 2560),
              (W.MODE_BF16, 640, 2560), (W.MODE_BF16, 10240, 320), (W.MODE_BF16, 320, 10240),
              (W.MODE_FP8, 2560, 16480), (W.MODE_FP8, 2560, 2560), (W.MODE_FP8, 6144, 2560),
              (W.MODE_NVFP4, 2560, 12800), (W.MODE_NVFP4, 6144, 2560)]
    names = {W.MODE_BF16: "bf16", W.MODE_FP8: "fp8", W.MODE_NVFP4: "nvfp4"}
    bpc = {W.MODE_BF16: 2.0, W.MODE_FP8: 1.0, W.MODE_NVFP4: 0.5625}
    out = {}
    for mode, k, n in shapes:
        nbytes = int(k * n * bpc[mode])
        copies = max(4, min(48, (1 << 30) // nbytes))
        made = [W.make_weight(mode, k, n, seed=300 + c) for c in range(copies)]
        ws = [w for (w, _) in made]
        scales = made[0][1].cpu().numpy() if mode == W.MODE_FP8 else None
        x = W.make_x(1, k, seed=7)
        op = SkinnyGemm([1], [n], w_scale=scales)
        outs = [torch.empty((1, n), dtype=torch.bfloat16, device="cuda")]
        med, best = time_graph_rotation(torch, lambda i: op(x, ws[i], out=outs), copies)
        line = {"weight_bytes": nbytes, "us": round(med, 3), "GBps": round(nbytes / med / 1e3, 1), "plan": op.describe(k, ws[0])}
        if ref is not None:
            sc_dev = [made[0][1]] if mode == W.MODE_FP8 else [None]
            rmed, _ = time_graph_rotation(torch, lambda i: ref.ref_skinny_gemm(x, [ws[i]], [mode], [n], sc_dev, [1], [n]), copies)
            line["reference_kernel_sm100a_us"] = round(rmed, 3)
        out[f"{names[mode]}_{k}x{n}"] = line
        del made, ws
        torch.cuda.empty_cache()
    return out


def bench_next_ops(torch):
    """The two further ops of the domain: SharedExpertDown (K 640 -> N 2560 with a 2560-long gate, the shape class
    the reference operator is tuned for: K <= 1024, rows 1 and 4; the reference's fused kernel beside it where it
    was compiled) and UntileHcBf16 (its one fixed shape; bytes in + out per second)."""
    import ctypes

    from qwen38_flash_ops_b200 import SharedExpertDown, UntileHcBf16
    from qwen38_flash_ops_b200 import workloads as W

    peak, _ = peaks()
    ref = _ref_util()
    lib = ref.ref_lib() if ref is not None else None
    if lib is not None and not hasattr(lib, "ref_shared_expert_down"):
        lib = None
    out = {"SharedExpertDown_640x2560_gate2560": {}, "UntileHcBf16_160x20480": {}}
    k, n, gk = 640, 2560, 2560
    names = {W.MODE_BF16: "bf16", W.MODE_FP8: "fp8", W.MODE_NVFP4: "nvfp4"}
    gen = torch.Generator(device="cuda").manual_seed(11)

    def bf16(*shape, scale=1.0):
        return (torch.randn(*shape, generator=gen, device="cuda") * scale).to(torch.bfloat16)

    for mode in (W.MODE_BF16, W.MODE_FP8, W.MODE_NVFP4):
        copies = 48
        made = [W.make_weight(mode, k, n, seed=500 + c) for c in range(copies)]
        ws = [w for (w, _) in made]
        scales = made[0][1] if mode == W.MODE_FP8 else None
        op = SharedExpertDown(w_scale=scales.cpu().numpy() if scales is not None else None)
        for m in (1, 4):
            g, u, gx, routed = bf16(m, k), bf16(m, k), bf16(m, gk), bf16(m, n)
            gw = bf16(gk, 1, scale=0.02)
            med, _ = time_graph_rotation(torch, lambda i: op(g, u, ws[i], gx, gw, routed), copies)
            line = {"us": round(med, 3)}
            if lib is not None:
                res = torch.empty_like(routed)
                vp = ctypes.c_void_p

                def ref_call(i):
                    err = lib.ref_shared_expert_down(vp(g.data_ptr()), vp(u.data_ptr()), m, k, vp(ws[i].data_ptr()), mode, n,
                                                     vp(scales.data_ptr() if scales is not None else None), vp(gx.data_ptr()), gk,
                                                     vp(gw.data_ptr()), vp(routed.data_ptr()), vp(res.data_ptr()), 0,
                                                     vp(torch.cuda.current_stream().cuda_stream))
                    assert err == 0

                rmed, _ = time_graph_rotation(torch, ref_call, copies)
                line["reference_kernel_sm100a_us"] = round(rmed, 3)
            out["SharedExpertDown_640x2560_gate2560"][f"{names[mode]}_M{m}"] = line
        del made, ws
        torch.cuda.empty_cache()
    src = [bf16(160, 20480) for _ in range(24)]
    for kind in (0, 1):
        op = UntileHcBf16(kind)
        dst = torch.empty((10240, 320) if kind == 0 else (320, 10240), dtype=torch.bfloat16, device="cuda")
        med, _ = time_graph_rotation(torch, lambda i: op(src[i], out=dst), len(src))
        nbytes = 2 * 160 * 20480 * 2
        out["UntileHcBf16_160x20480"][f"kind{kind}"] = {"us": round(med, 3), "GBps": round(nbytes / med / 1e3, 1),
                                                        "frac_of_measured_hbm": round(nbytes / med / 1e3 / peak, 4)}
    return out


def read_ceiling(torch):
    """GB/s of a read-only sweep (128-bit loads, nothing written) over 2 GiB, 16x L2: the streaming ceiling
    a weight stream is compared with, besides the copy bandwidth."""
    import ctypes

    from qwen38_flash_ops_b200 import _lib

    lib = _lib.load()
    nbytes = 2 << 30
    buf = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    buf.fill_(1)
    stream = torch.cuda.current_stream().cuda_stream

    def sweep():
        _lib.check(lib.qfg_stream_read_probe(buf.data_ptr(), nbytes, None, ctypes.c_void_p(stream)))

    ms = time_region(torch, sweep, 10, 3)
    del buf
    torch.cuda.empty_cache()
    return round(nbytes * 10 / ms / 1e6, 1)


def bench_argmax_and_dequant(torch):
    """ArgmaxRows over LM-head logits (1 / 4 / 8 / 64 rows, the reference's kernel beside it) and
    DequantWeightBf16 (bytes in + bytes out per second): device time per call from a CUDA graph of 20 calls."""
    from qwen38_flash_ops_b200 import ArgmaxRows, DequantWeightBf16
    from qwen38_flash_ops_b200 import workloads as W

    peak, _ = peaks()
    out = {"ArgmaxRows_bf16_151936": {}, "DequantWeightBf16": {}}
    ref = _ref_util()
    vocab = 151936
    op = ArgmaxRows()
    for rows in (1, 4, 8, 64):
        gen = torch.Generator(device="cuda").manual_seed(rows)
        x = (torch.randn((rows, vocab), generator=gen, device="cuda") * 1.43).to(torch.bfloat16)
        idx = torch.empty(rows, dtype=torch.int64, device="cuda")
        val = torch.empty(rows, dtype=torch.float32, device="cuda")
        med, best = time_graph_rotation(torch, lambda i: op(x, out=(idx, val)), 20)
        line = {"us": round(med, 3), "us_best": round(best, 3), "GBps": round(x.numel() * 2 / med / 1e3, 1)}
        if ref is not None:
            rmed, _ = time_graph_rotation(torch, lambda i: ref.ref_argmax_rows(x), 20)
            line["reference_kernel_sm100a_us"] = round(rmed, 3)
        out["ArgmaxRows_bf16_151936"][f"rows{rows}"] = line
    for label, mode, k, n in (("nvfp4_5120x17408", W.MODE_NVFP4, 5120, 17408), ("nvfp4_5120x151936", W.MODE_NVFP4, 5120, 151936),
                              ("fp8_5120x10240", W.MODE_FP8, 5120, 10240)):
        copies = max(2, min(16, -(-(1 << 30) // (k * n * 3))))
        ws, scale = [], None
        for c in range(copies):
            w, s_ = W.make_weight(mode, k, n, seed=50 + c)
            ws.append(w)
            scale = s_ if c == 0 else scale
        dq = DequantWeightBf16(n, w_scale=scale.cpu().numpy() if scale is not None else None)
        dst = torch.empty((k, n), dtype=torch.bfloat16, device="cuda")
        med, best = time_graph_rotation(torch, lambda i: dq(ws[i], out=[dst]), copies)
        moved = ws[0].numel() * ws[0].element_size() + k * n * 2
        out["DequantWeightBf16"][label] = {"us": round(med, 2), "GBps": round(moved / med / 1e3, 1),
                                           "frac_of_measured_hbm": round(moved / med / 1e3 / peak, 4),
                                           "bytes": moved}
        del ws, dst
        torch.cuda.empty_cache()
    return out


def _ref_util():
    """tests/_util when the reference project's kernels were compiled (oracle/_ref), else None."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    try:
        import _util as U
    except Exception:
        return None
    return U if U.ref_lib() is not None else None


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline(m, k, sample_cols, seed=11, reps=1):
    """The unfused chain on the host cores over the first `sample_cols` columns of the head."""
    import numpy as np

    from oracle import cpu as C
    from qwen38_flash_ops_b200 import packing as P

    # the launcher of multi-rank runs exports OMP_NUM_THREADS=1: the CPU arm uses every core it may run on
    C.set_num_threads(host_cores())

    rng = np.random.default_rng(seed)
    x = P.synth_x(rng, m, k)
    packed = rng.integers(0, 256, (k, sample_cols * 9 // 16), dtype=np.uint8)
    packed[:, sample_cols // 2:] = rng.integers(0x18, 0x40, (k, sample_cols // 16), dtype=np.uint8)
    C.chain_f32(2, x, packed[:, :], sample_cols)  # warm-up (thread pool, page faults)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        logits = C.chain_f32(2, x, packed, sample_cols)
        C.argmax_rows(0, logits)
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    nbytes = k * sample_cols * 9 // 16
    return {"value": round(nbytes / dt / 1e12, 6), "unit": UNIT, "cores": C.num_threads(), "kind": "port",
            "sample": f"dequantise + MatMul(FP32 acc) + ArgMax over {sample_cols} of 151936 columns, "
                      f"M={m}, K={k}: {nbytes / 1e6:.1f} MB of packed weights, median of {reps} passes "
                      f"({sum(times):.1f} s of host work), {dt * 1e3:.1f} ms per pass",
            "seconds": round(dt, 4)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from qwen38_flash_ops_b200 import workloads as W

    wl = W.CONFIGS[HEAD]
    m = args.rows
    sample_cols = wl.ns[0]
    runs = []
    for _ in range(args.warmup):
        cpu_baseline(m, wl.k, sample_cols)
    t_all = time.perf_counter()
    for _ in range(args.steps):
        runs.append(cpu_baseline(m, wl.k, sample_cols))
    total = time.perf_counter() - t_all
    secs = statistics.median(r["seconds"] for r in runs)
    nbytes = wl.k * sample_cols * 9 // 16
    value = nbytes / secs / 1e12
    base = dict(runs[0])
    base["value"] = round(value, 6)
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 6), "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(secs * 1e3, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 weights, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": HEAD, "rows": m, "sample_cols": sample_cols,
                       "note": "each step is the whole head once on the host cores; value = weight bytes / time"},
            "cpu_baseline": base,
            "e2e": {"value": round(value, 6), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": round(total, 2)}
    try:
        line["ref_kernel_sm100a"] = time_reference_gpu_kernels(m)
    except Exception as exc:  # no GPU, or the reference kernels were never compiled
        line["ref_kernel_sm100a"] = {"unavailable": str(exc)[:200]}
    print(json.dumps(line), flush=True)


def time_reference_gpu_kernels(m):
    """The reference project's own kernels (its generic launch configuration) recompiled for
    sm_100a, on the head workload: SkinnyGemm then ArgmaxRows, as the reference runs them."""
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device")
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import _util as U
    from qwen38_flash_ops_b200 import workloads as W

    if U.ref_lib() is None:
        raise RuntimeError("oracle/_ref/libref_kernels.so not built")
    wl = W.CONFIGS[HEAD]
    n = wl.ns[0]
    w, _ = W.make_weight(wl.mode, wl.k, n, seed=1)
    x = W.make_x(m, wl.k, seed=7)

    def call():
        y = U.ref_skinny_gemm(x, [w], [2], [n], [None], [1], [n])[0]
        U.ref_argmax_rows(y)

    ms = time_region(torch, call, 20, 5)
    us = ms * 1000.0 / 20
    return {"us_per_call": round(us, 2), "TBps": round(wl.weight_bytes / us / 1e6, 4), "rows": m,
            "what": "skinny::LaunchT<M,8,256,C,4> + LaunchArgmaxRows, unfused, eager launches"}


def run_ours(args):
    import torch

    from qwen38_flash_ops_b200 import _lib, packing
    from qwen38_flash_ops_b200 import workloads as W
    from qwen38_flash_ops_b200.lmhead_shard import ShardedLmHead

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    _lib.load()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    wl = W.CONFIGS[HEAD]
    m, k, n_total = args.rows, wl.k, wl.ns[0]
    c0, c1 = packing.shard_columns(n_total, world)[rank]
    n_local = c1 - c0
    shard, _ = W.make_weight(wl.mode, k, n_local, seed=100 + rank)
    head = ShardedLmHead(shard, n_local, c0)
    x = W.make_x(m, k, seed=7)
    if world > 1:
        dist.broadcast(x, 0)
    shard_bytes = k * n_local * 9 // 16
    total_bytes = wl.weight_bytes
    # the generated inputs, so that a run elsewhere can be checked to stream the same bytes (torch's CUDA generator,
    # seeds 100 + rank and 7); hashed on the host, outside every timed region
    import hashlib
    data_sha256 = {"x": hashlib.sha256(x.cpu().view(torch.int16).numpy()).hexdigest(),
                   "weights_rank0": hashlib.sha256(shard.cpu().numpy()).hexdigest() if rank == 0 else None}

    verified = None
    exchange_note = None
    if world > 1:
        ok = all(verify_sharded(torch, dist, head, xr, shard, n_local, c0, world) for xr in sharded_check_inputs(torch, dist, W, x, k))
        if not ok and head.peer is not None:
            # the in-kernel exchange failed its check on this machine: fall back to the collective and say so
            exchange_note = f"peer-memory exchange failed verification (status {head.peer.status()}); NCCL used instead"
            head = ShardedLmHead(shard, n_local, c0, exchange="nccl")
            ok = all(verify_sharded(torch, dist, head, xr, shard, n_local, c0, world) for xr in sharded_check_inputs(torch, dist, W, x, k))
        if not ok:
            raise SystemExit("sharded LM head disagrees with the fold of the per-rank unfused results")
        verified = "sharded step == fold of per-rank SkinnyGemm + ArgmaxRows, rows 1, 2, 4 and the timed batch"

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # kernel-resident timing: inputs already in HBM
    ms = time_region(torch, lambda: head.step(x), args.steps, args.warmup, dist)
    clocks = sampler.stop() if rank == 0 else None
    us_step = ms * 1000.0 / args.steps
    value = total_bytes / us_step / 1e6

    # inside the exchange of the last timed step, per rank: stores issued after the keys were ready, all ranks' words
    # seen after the stores; the slowest rank waits least, so the minimum over ranks of the wait is the latency of
    # the exchange itself and the rest of a rank's wait is time spent waiting for the slowest rank's kernel
    exchange_times = None
    exchange_alt = None
    if world > 1 and head.peer is not None:
        t_ready, t_sent, t_done = head.peer.times()
        mine = torch.tensor([(t_sent - t_ready) / 1000.0, (t_done - t_sent) / 1000.0], dtype=torch.float64, device="cuda")
        allt = torch.empty((world, 2), dtype=torch.float64, device="cuda")
        dist.all_gather_into_tensor(allt, mine)
        a = allt.cpu().numpy()
        exchange_times = {"store_us": {"min": round(float(a[:, 0].min()), 2), "max": round(float(a[:, 0].max()), 2)},
                          "wait_us": {"min": round(float(a[:, 1].min()), 2), "median": round(float(sorted(a[:, 1])[world // 2]), 2),
                                      "max": round(float(a[:, 1].max()), 2)},
                          "what": "last timed step, per rank, device timer: keys ready -> stores issued -> all ranks' words seen"}
        # the exchange the north star names, timed the same way: one NCCL all-gather of the keys and a fold kernel
        nccl_head = ShardedLmHead(shard, n_local, c0, exchange="nccl")
        ms_n = time_region(torch, lambda: nccl_head.step(x), args.steps, args.warmup, dist)
        exchange_alt = {"kind": "nccl_all_gather + fold kernel", "us_per_step": round(ms_n * 1000.0 / args.steps, 2),
                        "value": round(total_bytes / (ms_n * 1000.0 / args.steps) / 1e6, 4), "unit": UNIT}

    # the fused kernel alone on this rank (no collective): the roofline figure
    ms_k = time_region(torch, lambda: head.head(x, shard, n_local, col_offset=c0, out=head_out(head, m, torch)),
                       args.steps, args.warmup, dist)
    us_kernel = ms_k * 1000.0 / args.steps

    # end to end: host x -> device, fused head (+ all-gather + fold), index and value back to the host
    from qwen38_flash_ops_b200.lmhead_shard import HostLmHead

    host_head = HostLmHead(head, m, k)
    host_head.x_host.copy_(x.cpu())

    def e2e_step():
        host_head()  # pinned x -> device, fused head (+ all-gather + fold), idx / val -> pinned host, synchronise

    ih, vh = host_head()
    ref_idx, ref_val = head.step(x)
    if not (torch.equal(ih, ref_idx.cpu()) and torch.equal(vh, ref_val.cpu())):
        raise SystemExit("host-buffer LM head disagrees with the device-resident step")
    ms_e = time_region(torch, e2e_step, args.steps, args.warmup, dist)
    us_e2e = ms_e * 1000.0 / args.steps

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    peak, peak_kind = peaks()
    # DRAM bytes per launch from the ncu capture of this kernel on this workload (read + write sectors
    # over the packed weight bytes), scaled to the shard
    traffic = round(NCU_DRAM_BYTES_PER_WEIGHT_BYTE * shard_bytes)
    line = {
        "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(us_step / 1000.0, 6), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 weights, f16 x f16 -> f32 mma", "data": "synthetic",
        "data_sha256": data_sha256,
        "config": {"workload": HEAD, "rows": m, "k": k, "n": n_total, "weight_bytes": total_bytes,
                   "parallelism": f"vocab-sharded x{world}" if world > 1 else "single GPU",
                   "l2": "inputs larger than L2 (437.6 MB of weights per step" +
                         (f", {shard_bytes / 1e6:.1f} MB per rank)" if world > 1 else ")"),
                   "plan": describe_plan(head, k, shard)},
        "us_per_call": round(us_step, 2),
        "frac_of_8TBps": round(value / 8.0 / world, 4),
        "roofline": {"bound": "hbm", "achieved": round(shard_bytes / us_kernel / 1e3, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(shard_bytes / us_kernel / 1e3 / peak, 4), "traffic": traffic,
                     "peak_source": f"{peak_kind} copy bandwidth", "kernel": "SkinnyGemmKernel<NVFP4> (fused argmax)",
                     "kernel_us": round(us_kernel, 2), "algorithmic_bytes": shard_bytes},
        "e2e": {"value": round(total_bytes / us_e2e / 1e6, 4), "unit": UNIT, "h2d_bytes_per_step": x.numel() * 2,
                "d2h_bytes_per_step": m * 12, "us_per_step": round(us_e2e, 2)},
        "gpu_launches": args.steps * (1 if (world == 1 or head.peer is not None) else 2),
        "clocks": clocks,
    }
    if verified is not None:
        line["verified"] = verified
        line["config"]["exchange"] = ("keys stored into the peers' memory by the fused kernel (no collective launch)"
                                      if head.peer is not None else "NCCL all-gather + fold kernel")
        if exchange_note is not None:
            line["config"]["exchange_note"] = exchange_note
        if exchange_times is not None:
            line["exchange_times"] = exchange_times
        if exchange_alt is not None:
            line["exchange_alt"] = exchange_alt
        if head.peer is not None and head.peer.status() != 0:
            raise SystemExit("a wait for a peer's keys ran out during the run")
    if world == 1 and not args.skip_cpu:
        line["cpu_baseline"] = cpu_baseline(m, k, n_total, reps=40)
    if world == 1:
        # third denominator: the read-only streaming ceiling of this GPU, measured now
        ceiling = read_ceiling(torch)
        line["roofline"]["read_ceiling_gbs"] = ceiling
        line["roofline"]["frac_of_read_ceiling"] = round(shard_bytes / us_kernel / 1e3 / ceiling, 4)
        line["roofline"]["frac_of_8TBps"] = round(shard_bytes / us_kernel / 1e3 / 8000.0, 4)
    if world == 1 and not args.headline_only:
        line["all_configs"] = bench_small_configs(torch, quick=args.quick)
        line["all_configs"].update(bench_argmax_and_dequant(torch))
        if not args.quick:
            line["all_configs"]["model_shapes_scored_planner"] = bench_model_shapes(torch)
            line["all_configs"].update(bench_next_ops(torch))
        per_m = {}
        for mm in (1, 2, 4):
            xm = W.make_x(mm, k, seed=7)
            outm = head_out(head, mm, torch)
            if mm == m:
                usm = us_kernel  # the roofline measurement above is this case
            else:
                # after the sweeps above the GPU runs at its power cap for a while (SM clock 1.8-1.9 GHz instead of
                # 1.965, calls 5-10 % longer); like the headline, these cases are timed from an idle GPU
                time.sleep(1.0)
                msm = time_region(torch, lambda: head.head(xm, shard, n_local, col_offset=c0, out=outm), args.steps,
                                  args.warmup)
                usm = msm * 1000.0 / args.steps
            per_m[f"M{mm}"] = {"us": round(usm, 2), "GBps": round(shard_bytes / usm / 1e3, 1),
                               "frac_of_measured_hbm": round(shard_bytes / usm / 1e3 / peak, 4),
                               "frac_of_8TBps": round(shard_bytes / usm / 1e3 / 8000.0, 4)}
        line["all_configs"][HEAD] = per_m
        try:
            line["all_configs"][HEAD]["reference_kernel_sm100a"] = time_reference_gpu_kernels(m)
        except Exception as exc:
            line["all_configs"][HEAD]["reference_kernel_sm100a"] = {"unavailable": str(exc)[:200]}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def sharded_check_inputs(torch, dist, W, x, k):
    """The timed batch and batches of 1, 2 and 4 rows, identical on every rank."""
    batches = [x]
    for m in (1, 2, 4):
        xm = W.make_x(m, k, seed=70 + m)
        dist.broadcast(xm, 0)
        batches.append(xm)
    return batches


def verify_sharded(torch, dist, head, x, shard, n_local, c0, world):
    """Untimed: the sharded step against the fold of every rank's unfused SkinnyGemm + ArgmaxRows
    over its own columns (same Better order: larger value, then lower global index).  Returns the
    verdict agreed by all ranks."""
    from qwen38_flash_ops_b200 import ArgmaxRows, SkinnyGemm

    m = x.shape[0]
    idx, val = head.step(x)
    logits = SkinnyGemm([1], [n_local])(x, shard)[0]
    lidx, lval = ArgmaxRows()(logits)
    cand = torch.stack([lval.double(), (lidx + c0).double()], dim=1).contiguous()  # [m, 2]
    gathered = torch.empty((world, m, 2), dtype=torch.float64, device=x.device)
    dist.all_gather_into_tensor(gathered, cand)
    torch.cuda.synchronize()
    g = gathered.cpu().numpy()
    ok = True
    for r in range(m):
        best = max(range(world), key=lambda w: (g[w, r, 0], -g[w, r, 1]))
        ok = ok and int(g[best, r, 1]) == int(idx[r].item()) and float(g[best, r, 0]) == float(val[r].item())
    if head.peer is not None and head.peer.status() != 0:
        ok = False
    # every rank takes the same decision
    flag = torch.tensor([1 if ok else 0], device=x.device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return int(flag.item()) == 1


_OUT_CACHE = {}


def head_out(head, m, torch):
    if m not in _OUT_CACHE:
        _OUT_CACHE[m] = (torch.empty(m, dtype=torch.int64, device="cuda"),
                         torch.empty(m, dtype=torch.float32, device="cuda"),
                         torch.empty(m, dtype=torch.int64, device="cuda"))
    return _OUT_CACHE[m]


def describe_plan(head, k, shard):
    from qwen38_flash_ops_b200 import _lib

    n = shard.shape[1] * 16 // 9
    align = 16 if (shard.data_ptr() % 16 == 0 and shard.shape[1] % 16 == 0) else 8 if shard.shape[1] % 8 == 0 else 4
    p = _lib.plan_describe(_lib.QFG_UINT8, k, [n], align, spec="lmhead")
    return ",".join(f"{a}={b}" for a, b in p.items() if a != "seg_tiles")


def run_profile_case(args):
    """A few plain calls of one workload, for `ncu` (small launch count, no timing loop):
    python bench.py --profile-case C3_nvfp4_gate_up_5120x34816 --iters 3 [--rows M] [--copies C]"""
    import torch

    from qwen38_flash_ops_b200 import LmHeadArgmax, SkinnyGemm
    from qwen38_flash_ops_b200 import workloads as W

    wl = W.CONFIGS[args.profile_case]
    m = args.rows if args.rows else wl.m
    sets, scales = [], None
    for c in range(args.copies):
        ws, sc = [], []
        for i, n in enumerate(wl.ns):
            w, s_ = W.make_weight(wl.mode, wl.k, n, seed=1000 * c + i)
            ws.append(w)
            sc.append(s_)
        sets.append(ws)
        if c == 0 and wl.mode == W.MODE_FP8:
            scales = torch.cat(sc).cpu().numpy()
    x = W.make_x(m, wl.k, seed=7)
    if wl.fused_argmax:
        op = LmHeadArgmax()
        call = lambda i: op(x, sets[i % args.copies][0], wl.ns[0])
    else:
        seg_outs = [len(w) for w in wl.seg_widths]
        widths = [w for ws_ in wl.seg_widths for w in ws_]
        op = SkinnyGemm(seg_outs, widths, w_scale=scales, trigger=wl.trigger)
        call = lambda i: op(x, *sets[i % args.copies])
    torch.cuda.synchronize()
    for i in range(args.iters):
        call(i)
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": args.profile_case, "rows": m, "iters": args.iters, "copies": args.copies,
                      "weight_bytes": wl.weight_bytes}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=4, help="rows of x per step (1-4 in the benchmark)")
    ap.add_argument("--headline-only", action="store_true", help="skip the C1-C4 sweep")
    ap.add_argument("--quick", action="store_true", help="fewer weight copies in the C1-C4 sweep")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--profile-case", default=None, help="run a few plain calls of this workload (for ncu) and exit")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--copies", type=int, default=3, help="weight copies rotated through by --profile-case")
    args = ap.parse_args()
    if args.profile_case:
        if "--rows" not in sys.argv:
            args.rows = 0
        run_profile_case(args)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        if args.steps > 20:
            args.steps = 20
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
