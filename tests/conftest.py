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


# ---------------------------------------------------------------------------------------------
# Guard zones.  compute-sanitizer is not available for these runs, so out-of-bounds stores are
# caught the plain way: every output the parity helpers hand to the library sits between two
# zones filled with a canary bit pattern (a NaN payload no kernel produces), the output itself
# starts out as the same pattern (a stale buffer, allocator.rs:61-66), and after the call the
# zones must be untouched and -- unless the call accumulates -- no canary may be left inside.
GUARD_FLOATS = 1024            # 4 KiB on each side; keeps the output's 256-byte alignment
CANARY = 0x7FC0BEEF


class Guarded:
    """A device tensor of `shape` with canary-filled guard zones before and after it."""

    def __init__(self, F, shape, init=None, misalign=0):
        import torch
        self.n = int(np.prod(shape)) if len(shape) else 1
        self.lo = GUARD_FLOATS + misalign          # misalign (floats) moves the output off its 16-byte alignment
        self.raw = torch.full((self.n + 2 * GUARD_FLOATS + misalign,), CANARY, dtype=torch.int32, device="cuda")
        flat = self.raw.view(torch.float32)[self.lo:self.lo + max(self.n, 1)]
        if init is not None:
            flat[:self.n].copy_(torch.from_numpy(np.ascontiguousarray(init, np.float32).ravel()))
        self.tensor = F.DeviceTensor(flat, shape)

    def check(self, what="output", fully_written=True):
        import torch
        torch.cuda.synchronize()
        before = self.raw[:self.lo]
        after = self.raw[self.lo + self.n:]
        assert bool((before == CANARY).all()), f"{what}: store below the buffer"
        assert bool((after == CANARY).all()), f"{what}: store past the end of the buffer"
        if fully_written and self.n:
            inside = self.raw[self.lo:self.lo + self.n]
            assert not bool((inside == CANARY).any()), f"{what}: elements left unwritten"


def regression_bound_3xtf32(k):
    """What the 3xTF32 path actually delivers against the sequential-f32 CPU loop, as a relative Frobenius
    error: ~1e-6 from the split (the lo parts are themselves cut to TF32) plus the CPU loop's own
    accumulation rounding, which grows like sqrt(K) * 2^-24.  A single-pass TF32 product sits near 3e-4,
    two orders of magnitude above this at every K the tests use, so a broken split cannot hide under it."""
    return 5e-6 + 1.2e-7 * float(np.sqrt(max(int(k), 1)))
