"""pytest configuration: the `gpu` marker and shared helpers."""

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"

# north-star tolerances: rel-L2 against the reference / oracle
REL_L2_TOL = {
    torch.float32: 1e-5, torch.complex64: 1e-5,
    torch.float64: 1e-12, torch.complex128: 1e-12,
    np.dtype(np.float32): 1e-5, np.dtype(np.complex64): 1e-5,
    np.dtype(np.float64): 1e-12, np.dtype(np.complex128): 1e-12,
}
# element-wise tolerance of the reference's own accuracy tests
# (tests/pytest/accuracy_utils.py:17-30: rtol = atol)
ALLCLOSE_TOL = {
    np.dtype(np.float32): 1.3e-6, np.dtype(np.complex64): 1.3e-6,
    np.dtype(np.float64): 1e-7, np.dtype(np.complex128): 1e-7,
}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Group the flat 'case/field' keys of an .npz fixture into {case: {field: array}}."""
    raw = np.load(GOLDEN_DIR / name)
    cases = {}
    for key in raw.files:
        case, field = key.split("/")
        cases.setdefault(case, {})[field] = raw[key]
    return cases


@pytest.fixture(scope="session")
def spmv_golden():
    return load_golden("spmv_reference.npz")


@pytest.fixture(scope="session")
def spmm_golden():
    return load_golden("spmm_reference.npz")
