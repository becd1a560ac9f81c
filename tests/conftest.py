import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    # the product path must be the native library; fail loudly if it is missing
    from qwen38_flash_ops_b200 import _lib

    _lib.load()
    return torch.device("cuda:0")


def to_dev(arr: np.ndarray, kind: str):
    """numpy bit patterns -> CUDA tensor of the element type the op expects."""
    import torch

    t = torch.from_numpy(np.ascontiguousarray(arr)).cuda()
    if kind == "bf16":
        return t.view(torch.int16).view(torch.bfloat16)
    if kind == "fp16":
        return t.view(torch.int16).view(torch.float16)
    if kind == "fp8":
        return t.view(torch.float8_e4m3fn)
    return t


def bits(t) -> np.ndarray:
    """CUDA BF16/FP16 tensor -> uint16 bit patterns on the host."""
    import torch

    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
