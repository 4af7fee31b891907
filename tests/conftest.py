"""Shared fixtures: markers, golden-vector loaders, error metrics."""
import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


class Golden:
    """One golden .npz: ``cases`` (list of dicts) and array lookup by key."""

    def __init__(self, name):
        self._z = np.load(GOLDEN / name)
        self.cases = json.loads(bytes(self._z["__cases__"]).decode())

    def __getitem__(self, key):
        return self._z[key]


@pytest.fixture(scope="session")
def golden_parity():
    return Golden("parity.npz")


@pytest.fixture(scope="session")
def golden_channel():
    return Golden("channel_parity.npz")


@pytest.fixture(scope="session")
def golden_extra():
    return Golden("spec_extra.npz")


def max_rel_l2(a, b):
    """Largest per-vector ||a-b|| / ||b|| (the reference tests' maxRelativeDifference,
    Tests/PITCHTests/TestSupport.swift:53-96); zero reference vectors compare absolutely."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    num = np.sqrt(((a - b) ** 2).sum(axis=1))
    den = np.sqrt((b ** 2).sum(axis=1))
    return float(np.max(num / np.where(den > 0, den, 1.0)))


def mean_rel_err(x, y):
    """Mean of ||x-y||^2/||x||^2 over vectors with non-zero norm."""
    x = np.asarray(x, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    den = (x ** 2).sum(axis=1)
    keep = den > 0
    return float((((x - y) ** 2).sum(axis=1)[keep] / den[keep]).mean())
