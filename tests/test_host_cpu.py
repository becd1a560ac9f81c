"""CPU-side checks of the C-ABI library and the host logic: the library loads and exports every
symbol the header declares, attribute validation refuses bad nodes before any CUDA call, the
launch planner's invariants hold, and the product fails loudly without a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

from qwen38_flash_ops_b200 import _lib
from qwen38_flash_ops_b200 import lmhead_shard as LS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "qfg.h")).read()
    declared = set(re.findall(r"QFG_API\s+[\w\s\*]+?\b(qfg_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.EXPORTS)
    lib = _lib.load()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.qfg_version().decode().endswith("sm_100a")


def _create(seg_outs, widths, scale=None, trigger=0):
    lib = _lib.load()
    h = ctypes.c_void_p()
    so, wi = _lib.i64_array(seg_outs), _lib.i64_array(widths)
    code = lib.qfg_skinny_gemm_create(so, len(seg_outs), wi, len(widths), None, 0, trigger, ctypes.byref(h))
    return code, lib.qfg_last_error().decode(), h


@pytest.mark.parametrize("seg_outs,widths", [
    ([], []),                       # no weight
    ([1, 1, 1, 1, 1], [8] * 5),     # more than four weights
    ([2], [64]),                    # seg_outs do not add up to len(widths)
    ([5, 4], [8] * 9),              # more than eight outputs
    ([1], [0]),                     # empty output
    ([0], []),
])
def test_bad_attributes_are_refused_before_any_cuda_call(seg_outs, widths):
    code, msg, h = _create(seg_outs, widths)
    assert code == _lib.QFG_INVALID_ARGUMENT and not h.value
    assert "bad seg_outs/widths" in msg


def test_dequant_attribute_validation():
    lib = _lib.load()
    h = ctypes.c_void_p()
    assert lib.qfg_dequant_create(100, 0, None, 0, None, 0, ctypes.byref(h)) == _lib.QFG_INVALID_ARGUMENT
    assert "multiple of 8" in lib.qfg_last_error().decode()
    w = _lib.i64_array([64, 32])
    assert lib.qfg_dequant_create(128, 0, w, 2, None, 0, ctypes.byref(h)) == _lib.QFG_INVALID_ARGUMENT
    assert lib.qfg_dequant_create(128, 4, None, 0, None, 0, ctypes.byref(h)) == _lib.QFG_INVALID_ARGUMENT


def test_argmax_argument_validation_needs_no_device():
    lib = _lib.load()
    assert lib.qfg_argmax_rows(_lib.QFG_INT64, None, 1, 8, None, None, None) == _lib.QFG_INVALID_ARGUMENT
    assert lib.qfg_argmax_rows(_lib.QFG_FLOAT, None, 0, 8, None, None, None) == _lib.QFG_OK       # rows == 0
    assert lib.qfg_argmax_rows(_lib.QFG_FLOAT, None, 2, 0, None, None, None) == _lib.QFG_INVALID_ARGUMENT


def test_no_cpu_fallback():
    """Without a GPU a valid node cannot be created: the product has no CPU path."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    code, msg, h = _create([1], [128])
    assert code != _lib.QFG_OK and not h.value


SHAPES = [
    (_lib.QFG_BFLOAT16, 5120, [5120], 16),
    (_lib.QFG_FLOAT8E4M3FN, 5120, [8192, 1024, 1024], 16),
    (_lib.QFG_UINT8, 5120, [17408, 17408], 16),
    (_lib.QFG_UINT8, 17408, [5120], 16),
    (_lib.QFG_UINT8, 5120, [151936], 8),
    (_lib.QFG_UINT8, 5120, [19072], 8),
    (_lib.QFG_BFLOAT16, 320, [10240], 16),
    (_lib.QFG_BFLOAT16, 10240, [320, 4], 8),
    (_lib.QFG_FLOAT8E4M3FN, 256, [100], 4),
    (_lib.QFG_UINT8, 64, [64], 4),
]


@pytest.mark.parametrize("dtype,k,n,align", SHAPES)
def test_plan_invariants(dtype, k, n, align):
    cpw = {_lib.QFG_BFLOAT16: 64, _lib.QFG_FLOAT8E4M3FN: 128, _lib.QFG_UINT8: 128}[dtype]
    for sms in (148, 132, 16):
        p = _lib.plan_describe(dtype, k, n, align, sms)
        assert p["wn"] * p["wk"] * 32 == p["threads"] <= 640
        assert 1 <= p["cluster"] <= 8 and 2 <= p["stages"] <= 8
        assert p["smem"] <= 227 * 1024
        assert sum(p["seg_tiles"]) == p["tiles"] and p["ctas"] == p["tiles"] * p["cluster"]
        for width, tiles in zip(n, p["seg_tiles"]):
            granules = -(-width // p["gran"])
            assert 1 <= tiles <= granules
            widest = -(-granules // tiles) * p["gran"]
            assert widest <= p["wn"] * cpw * p["wide"], "a tile must fit the CTA's columns"
        if sms == 148 and sum(n) * k > 2 ** 24:
            assert p["ctas"] >= 0.8 * 148, "a large shape must cover (nearly) every SM"


def test_plan_override_and_errors():
    p = _lib.plan_describe(_lib.QFG_UINT8, 5120, [17408], 16, 148, "direct=0,wn=4,wk=2,cluster=2,ctas=296,stages=5,ks=2")
    assert (p["direct"], p["wn"], p["wk"], p["cluster"], p["stages"], p["ks"], p["ctas"]) == (0, 4, 2, 2, 5, 2, 296)
    p = _lib.plan_describe(_lib.QFG_UINT8, 5120, [17408], 16, 148, "wn=4,wk=4,cluster=2,ctas=148")
    assert (p["direct"], p["threads"], p["ctas"]) == (1, 512, 148)
    # shapes the register-streaming kernel cannot take fall back to the ring kernel
    assert _lib.plan_describe(_lib.QFG_BFLOAT16, 256, [132], 8)["direct"] == 0
    assert _lib.plan_describe(_lib.QFG_UINT8, 256, [192], 4)["direct"] == 0
    with pytest.raises(_lib.QfgError):
        _lib.plan_describe(_lib.QFG_UINT8, 256, [192], 4, 148, "direct=1")
    with pytest.raises(_lib.QfgError):
        _lib.plan_describe(_lib.QFG_UINT8, 5120, [17408], 16, 148, "wn=11")
    with pytest.raises(_lib.QfgError):
        _lib.plan_describe(_lib.QFG_UINT8, 5120, [17408], 16, 148, "bogus=1")
    with pytest.raises(_lib.QfgError):
        _lib.plan_describe(_lib.QFG_FLOAT, 5120, [17408], 16, 148)


def test_key_pack_orders_like_argmax():
    from oracle import oracle as O

    vals = np.array([1.5, 1.5, -0.0, 0.0, -3.0, np.inf, -np.inf, np.nan, np.nan, 1e-40], np.float32)
    idxs = np.array([7, 3, 10, 11, 0, 5, 6, 9, 8, 2], np.int64)
    keys = LS.pack_key(vals, idxs)
    for i in range(len(vals)):
        for j in range(len(vals)):
            if i != j:
                assert (keys[i] > keys[j]) == O.better(vals[i], idxs[i], vals[j], idxs[j]), (i, j)
    v, ix = LS.unpack_key(keys)
    assert np.array_equal(ix, idxs)
    assert np.array_equal(np.isnan(v), np.isnan(vals))
    ok = ~np.isnan(vals)
    assert np.array_equal(v[ok], vals[ok])
