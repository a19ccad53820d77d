"""Shared fixtures.  Tests that need a B200 carry the ``gpu`` marker."""

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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name)))


def bf16_from_bits(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


@pytest.fixture(scope="session")
def consts():
    z = load_golden("constants.npz")
    # QR hands back column-major factors; make every constant row-major once
    return {k: torch.from_numpy(np.ascontiguousarray(v)).contiguous() for k, v in z.items()}
