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


# Where the GPU tests leave their parity figures (one JSON object per line), if that folder exists.
RECORD_DIR = os.environ.get("MDB200_RECORD_DIR", os.path.join(ROOT, "gpurun_out"))


def record_parity(name: str, **figures) -> None:
    """Parity figures of a test: printed, and appended to ``parity_tests.jsonl`` in the records folder."""
    import json
    line = json.dumps(dict(test=name, **figures))
    print("PARITY " + line)
    if os.path.isdir(RECORD_DIR):
        with open(os.path.join(RECORD_DIR, "parity_tests.jsonl"), "a") as f:
            f.write(line + "\n")


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
