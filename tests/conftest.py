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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def bits_of(t: torch.Tensor) -> np.ndarray:
    """Raw bytes/words of a 1- or 2-byte-element tensor as numpy unsigned ints."""
    t = t.detach().cpu().contiguous()
    if t.element_size() == 1:
        return t.view(torch.uint8).numpy()
    return t.view(torch.int16).numpy().view(np.uint16)


@pytest.fixture(scope="session")
def golden_quant():
    return np.load(os.path.join(GOLDEN, "quant.npz"))


@pytest.fixture(scope="session")
def golden_mm():
    return np.load(os.path.join(GOLDEN, "mm.npz"))


@pytest.fixture(scope="session")
def golden_attn():
    return np.load(os.path.join(GOLDEN, "attn.npz"))
