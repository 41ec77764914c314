"""GPU: the allocation-free bias-add backward against the regular entry point.

Some hosts of this library may not let it allocate device memory: the reference's tensor store
owns the device's memory through its own allocator, and a training loop cannot absorb the
device-wide synchronisation of cudaMalloc / cudaFree in the middle of a step.  For them
``mni_b200_add_bias_bwd_noalloc`` keeps its partial sums in a fixed array inside the library.
This file is collected last on purpose, so a failure here cannot hide the other tests' results;
it passes on its own in a fresh process as well (the entry point does its own per-device set-up).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import framework_b200 as F
    F._lib.lib()
    return F


def _both(F, dy_np, accumulate_into=None):
    """Runs the regular and the allocation-free entry point through the C ABI on the same input."""
    import torch
    from framework_b200.tensor import current_stream
    lib = F._lib.lib()
    rows, n = dy_np.shape
    dy = F.DeviceTensor.from_numpy(dy_np)
    outs = []
    for fn in (lib.mni_b200_add_bias_bwd, lib.mni_b200_add_bias_bwd_noalloc):
        d_y = F.DeviceTensor(torch.full((rows * n,), float("nan"), device="cuda"), (rows, n))
        if accumulate_into is None:
            dbias = F.DeviceTensor(torch.full((n,), float("nan"), device="cuda"), (n,))
            flags = 0
        else:
            dbias = F.DeviceTensor.from_numpy(accumulate_into)
            flags = F._lib.ACCUMULATE_DBIAS
        F._lib.check(fn(dy.ptr, d_y.ptr, dbias.ptr, rows, n, flags, current_stream()))
        torch.cuda.synchronize()
        outs.append((d_y.numpy(), dbias.numpy()))
    return outs


def test_matches_regular_entry_point_on_two_calls_in_a_row(F):
    rng = np.random.default_rng(31)
    # Two calls back to back with different shapes: the second one finds the first one's
    # partial sums still in the shared array and must not be affected by them.
    for rows, n in ((4096, 4096), (777, 130)):
        dy = rng.standard_normal((rows, n), dtype=np.float32)
        (ref_dy, ref_db), (got_dy, got_db) = _both(F, dy)
        assert np.array_equal(got_dy, dy) and np.array_equal(ref_dy, dy)
        # same kernels, same summation order: identical; the parity bound of the suite is the gate
        bound = 1e-5 * rows * float(np.abs(dy).max())
        assert float(np.max(np.abs(got_db - ref_db))) <= bound
        exact = dy.astype(np.float64).sum(0)
        assert float(np.max(np.abs(got_db - exact))) <= bound
    base = rng.standard_normal(130, dtype=np.float32)
    dy = rng.standard_normal((50, 130), dtype=np.float32)
    (_, ref_db), (_, got_db) = _both(F, dy, accumulate_into=base)
    assert float(np.max(np.abs(got_db - ref_db))) <= 1e-5 * 50 * float(np.abs(dy).max())


def test_device_memory_does_not_move_and_results_are_bitwise_equal(F):
    """What the entry point is for: after the library's own scratch has been released, so that the regular
    entry point would have to cudaMalloc, a call through the allocation-free one leaves the device's free
    memory exactly where it was.  The outputs are bitwise those of the regular entry point (same kernels,
    same summation order), also when a call on other data ran in between and left its partial sums in the
    shared array."""
    import torch
    from framework_b200.tensor import current_stream
    lib = F._lib.lib()
    rng = np.random.default_rng(33)
    rows, n = 6000, 1536
    dy_np = rng.standard_normal((rows, n), dtype=np.float32)
    other_np = rng.standard_normal((900, 2048), dtype=np.float32)
    dy, other = F.DeviceTensor.from_numpy(dy_np), F.DeviceTensor.from_numpy(other_np)
    outs = {k: torch.full((n,), float("nan"), device="cuda") for k in ("first", "again", "regular")}
    other_out = torch.empty(2048, device="cuda")
    # Warm-up on a small input, so that the kernels' code is resident (a first launch loads it, which takes device
    # memory of its own) and the entry point's per-device set-up has run -- what a caller does at start-up.
    warm = torch.ones(64 * 8, device="cuda")
    warm_out = torch.empty(8, device="cuda")
    F._lib.check(lib.mni_b200_add_bias_bwd_noalloc(warm.data_ptr(), None, warm_out.data_ptr(), 64, 8, 0, current_stream()))
    F._lib.check(lib.mni_b200_add_bias_bwd(warm.data_ptr(), None, warm_out.data_ptr(), 64, 8, 0, current_stream()))
    torch.cuda.synchronize()
    F._lib.check(lib.mni_b200_release())                 # drop the growable scratch: a regular call must allocate now
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    F._lib.check(lib.mni_b200_add_bias_bwd_noalloc(dy.ptr, None, outs["first"].data_ptr(), rows, n, 0, current_stream()))
    F._lib.check(lib.mni_b200_add_bias_bwd_noalloc(other.ptr, None, other_out.data_ptr(), 900, 2048, 0, current_stream()))
    F._lib.check(lib.mni_b200_add_bias_bwd_noalloc(dy.ptr, None, outs["again"].data_ptr(), rows, n, 0, current_stream()))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "device memory moved during allocation-free calls"
    F._lib.check(lib.mni_b200_add_bias_bwd(dy.ptr, None, outs["regular"].data_ptr(), rows, n, 0, current_stream()))
    torch.cuda.synchronize()
    first, again, regular = (outs[k].cpu().numpy() for k in ("first", "again", "regular"))
    assert np.array_equal(first, regular) and np.array_equal(again, regular)
    assert float(np.max(np.abs(regular - dy_np.astype(np.float64).sum(0)))) <= 1e-5 * rows * float(np.abs(dy_np).max())
    assert float(np.max(np.abs(other_out.cpu().numpy() - other_np.astype(np.float64).sum(0)))) <= 1e-5 * 900 * 6.0


def test_refuses_sizes_beyond_the_built_in_scratch(F):
    import torch
    from framework_b200.tensor import current_stream
    lib = F._lib.lib()
    n = 300_000                       # one slab of partial sums = 1.2 MB > 1 MiB
    dy = torch.zeros(2 * n, device="cuda")
    db = torch.zeros(n, device="cuda")
    rc = lib.mni_b200_add_bias_bwd_noalloc(dy.data_ptr(), None, db.data_ptr(), 2, n, 0, current_stream())
    assert rc == 7, "expected MNI_B200_ERR_WORKSPACE"
    assert b"built-in scratch" in lib.mni_b200_last_error()
    # the regular entry point takes the same size
    F._lib.check(lib.mni_b200_add_bias_bwd(dy.data_ptr(), None, db.data_ptr(), 2, n, 0, current_stream()))
    torch.cuda.synchronize()
