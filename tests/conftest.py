"""Shared pytest configuration: the `gpu` marker, import paths, golden-fixture loader."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "tensor-product-attention-jax_b200")
for p in (ROOT, PKG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    """Return {case: {field: array}} from tests/golden/<name>.npz."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cases = {}
    for key in z.files:
        case, field = key.rsplit("/", 1)
        cases.setdefault(case, {})[field] = z[key]
    return cases


@pytest.fixture(scope="session")
def golden_fwd():
    return load_golden("fwd_matrix")


@pytest.fixture(scope="session")
def golden_ring():
    return load_golden("ring_matrix")


@pytest.fixture(scope="session")
def golden_extra():
    return load_golden("extra")
