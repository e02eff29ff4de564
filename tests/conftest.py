"""Shared pytest configuration: path set-up, the ``gpu`` marker and golden-vector loading."""

import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "towards-batched-activation-sparsity_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the reference's own Python functions plus the seeds of their inputs."""
    g = ROOT / "tests" / "golden"
    data = np.load(g / "reference_outputs.npz")
    meta = json.loads((g / "reference_outputs.json").read_text())
    return data, meta
