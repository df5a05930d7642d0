import importlib
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def mdb():
    """The package (its directory name has a hyphen)."""
    return importlib.import_module("mineru-diffusion_b200")


def load_golden(name: str) -> dict:
    return dict(np.load(os.path.join(GOLDEN, name)))


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns -> bf16 tensor."""
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def ulp_diff_bf16(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 units-in-the-last-place between two bf16 tensors."""
    def key(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(a) - key(b)).abs()
