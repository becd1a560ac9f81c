"""B200 (sm_100a) implementation of the `qwen.fused_gemm` decode weight-streaming path:
SkinnyGemm (M <= 8 rows per pass; BF16 / FP8 E4M3FN / block-16 NVFP4 weights), ArgmaxRows,
DequantWeightBf16 and the fused, N-shardable LM head.  The compute lives in libqfg_b200.so
(C ABI in include/qfg.h); this package is the Python mirror of the operator interface."""
from . import packing  # noqa: F401
from ._lib import QfgError, load  # noqa: F401


def __getattr__(name):
    # the operator classes need torch; import them lazily so packing / loading work without it
    if name in ("SkinnyGemm", "SharedExpertDown", "ArgmaxRows", "DequantWeightBf16", "UntileHcBf16", "LmHeadArgmax",
                "lmhead_combine"):
        from . import ops

        return getattr(ops, name)
    if name == "ShardedLmHead":
        from .lmhead_shard import ShardedLmHead

        return ShardedLmHead
    raise AttributeError(name)
