import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def golden():
    with open(os.path.join(ROOT, "tests", "golden", "reference_kat.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def oracle():
    import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def F():
    """The package with its CUDA library loaded; a GPU test without a device fails, it does not skip."""
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import framework_b200 as pkg
    pkg._lib.lib()
    return pkg


def tol_3xtf32(k, a, b):
    """Acceptance bound of the default precision mode: 1e-5 * K * max|a| * max|b|."""
    ma = float(np.max(np.abs(a))) if np.size(a) else 0.0
    mb = float(np.max(np.abs(b))) if np.size(b) else 0.0
    return 1e-5 * max(int(k), 1) * ma * mb + 1e-30


def rel_fro(x, ref):
    d = np.linalg.norm((np.asarray(x, np.float64) - np.asarray(ref, np.float64)).ravel())
    n = np.linalg.norm(np.asarray(ref, np.float64).ravel())
    return d / max(n, 1e-30)
