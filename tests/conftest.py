"""Shared test set-up: marker registration, import path, seeded EXL3 inputs."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped, not failed, where no device is visible and -m gpu was not asked for."""
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def seeded_trellis(seed: int, kt: int, nt: int, K: int) -> np.ndarray:
    """Uniform-random trellis words, uint16 [kt, nt, 16K], from numpy's PCG64 (same generator as the fixtures)."""
    rng = np.random.default_rng(seed)
    return rng.integers(0, 65536, size=(kt, nt, 16 * K), dtype=np.uint16)


def seeded_signs(seed: int, n: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "exl3_golden.npz")
    return np.load(path)
