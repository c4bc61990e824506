"""Shared pytest configuration: the ``gpu`` marker and import paths."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device and the built libpare_b200.so")


@pytest.fixture(scope="session")
def golden():
    """Loader for the committed fixtures produced by running the reference (tests/golden/generate.py)."""
    def load(name: str):
        return np.load(GOLDEN / name)
    return load


@pytest.fixture(scope="session")
def cuda_lib():
    """The loaded CUDA library; GPU tests fail (not skip) when it is missing."""
    import torch
    from pare_b200.kernels import _lib

    assert torch.cuda.is_available(), "gpu-marked test run without a CUDA device"
    return _lib.lib()
