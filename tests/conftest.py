"""Shared test setup: the ``gpu`` marker, import paths, and the golden fixtures."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG_PARENT = ROOT / "semantic-block-sparse-attention_b200"
for p in (str(ROOT), str(PKG_PARENT)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "reference_golden.npz")
