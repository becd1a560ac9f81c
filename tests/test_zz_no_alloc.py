"""The allocation-free LM-head entry point (qfg_lmhead_compute_static), called through the C ABI.

It exists for hosts that cannot give the library device memory: its scratch is an array built
into the library instead of a caller-provided workspace.  The result must be bit-identical to the
regular entry point, on two calls in a row (the second call finds the array as the first left
it), and row counts beyond the built-in limit must be refused.  This file sorts last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import to_dev
from qwen38_flash_ops_b200 import LmHeadArgmax, QfgError, _lib
from qwen38_flash_ops_b200 import packing as P

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_entry_point(cuda):
    rng = np.random.default_rng(2024)
    K, N = 640, 128 * 21
    pk = to_dev(P.pack_nvfp4(P.synth_weight(rng, K, N)), "u8")
    head = LmHeadArgmax()
    lib = _lib.load()
    assert lib.qfg_lmhead_static_max_rows() == 8
    for call, m in enumerate((4, 8)):
        x = to_dev(P.synth_x(rng, m, K), "bf16")
        ref_idx, ref_val, ref_key = head(x, pk, N, col_offset=7 * call)
        out = (torch.full((m,), -1, dtype=torch.int64, device="cuda"), torch.zeros(m, device="cuda"),
               torch.zeros(m, dtype=torch.int64, device="cuda"))
        idx, val, key = head.call_static(x, pk, N, col_offset=7 * call, out=out)
        torch.cuda.synchronize()
        assert torch.equal(idx, ref_idx), f"call {call}"
        assert torch.equal(val.view(torch.int32), ref_val.view(torch.int32)), f"call {call}"
        assert torch.equal(key, ref_key), f"call {call}"
    # more rows than the built-in array holds: a clear refusal, nothing launched
    x9 = to_dev(P.synth_x(rng, 9, K), "bf16")
    with pytest.raises(QfgError) as e:
        head.call_static(x9, pk, N)
    assert e.value.code == _lib.QFG_INVALID_ARGUMENT and "at most 8 rows" in str(e.value)
    # and the entry point still works afterwards
    x1 = to_dev(P.synth_x(rng, 1, K), "bf16")
    a = head.call_static(x1, pk, N)
    b = head(x1, pk, N)
    torch.cuda.synchronize()
    assert torch.equal(a[0], b[0]) and torch.equal(a[2], b[2])


def test_static_scratch_on_a_side_stream_and_a_width_the_workspace_entry_would_share(cuda):
    """594 column groups on 148 SMs leave two groups over: qfg_lmhead_compute shares them among its CTAs
    (partial sums in the workspace), the static entry point has no room for that and runs the plain launch
    shape, whose logits are SkinnyGemm's.  So its winners equal ArgmaxRows(SkinnyGemm(x)) bit for bit, on a
    non-blocking side stream as well as on the default one."""
    from qwen38_flash_ops_b200 import ArgmaxRows, SkinnyGemm

    rng = np.random.default_rng(77)
    K, N, m = 256, 128 * (148 * 4 + 2), 2
    pk = to_dev(P.pack_nvfp4(P.synth_weight(rng, K, N)), "u8")
    x = to_dev(P.synth_x(rng, m, K), "bf16")
    eidx, eval_ = ArgmaxRows()(SkinnyGemm([1], [N])(x, pk)[0])
    head = LmHeadArgmax()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    for stream in (torch.cuda.current_stream(), side, side):
        with torch.cuda.stream(stream):
            idx, val, _ = head.call_static(x, pk, N)
        stream.synchronize()
        assert torch.equal(idx, eidx) and torch.equal(val.view(torch.int32), eval_.view(torch.int32))
