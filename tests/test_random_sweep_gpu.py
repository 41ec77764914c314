"""Seeded random sweep of the matmul path against the CPU restatement: shapes from 1 to a few hundred in
every dimension, batch prefixes with and without broadcasting, transposed / permuted operand views, bias,
forced K splits and the single-pass mode.  Forty cases forward and backward; every case is checked against
the acceptance bound of its precision mode."""
import numpy as np
import pytest

from conftest import rel_fro, tol_3xtf32

pytestmark = pytest.mark.gpu

SIZES = [1, 2, 3, 5, 8, 16, 31, 33, 64, 65, 100, 128, 129, 200, 256, 300, 384, 520]


def _case(seed):
    rng = np.random.default_rng(1000 + seed)
    m, k, n = (int(rng.choice(SIZES)) for _ in range(3))
    kind = int(rng.integers(0, 5))
    if kind == 0:
        ba, bb = (), ()
    elif kind == 1:
        ba = bb = (int(rng.integers(1, 4)),)
    elif kind == 2:
        ba, bb = (int(rng.integers(2, 5)),), ()                  # broadcast weight
    elif kind == 3:
        ba, bb = (1, int(rng.integers(2, 4))), (int(rng.integers(2, 4)), 1)   # two-sided broadcast
    else:
        ba, bb = (), (int(rng.integers(2, 4)),)
    ta, tb = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
    flags = 0
    if rng.integers(0, 4) == 0:
        flags |= int(rng.integers(2, 5)) << 16                   # forced K split
    fast = bool(rng.integers(0, 6) == 0)
    bias = bool(rng.integers(0, 2))
    return rng, (m, k, n), ba, bb, ta, tb, flags, fast, bias


@pytest.mark.parametrize("seed", range(40))
def test_random_case(F, oracle, seed):
    rng, (m, k, n), ba, bb, ta, tb, flags, fast, bias = _case(seed)
    H = oracle.HostTensor
    # storage layouts: a transposed operand is stored [.., k, m] and viewed through a stride-only permute
    a_store = rng.standard_normal(ba + ((k, m) if ta else (m, k)), dtype=np.float32)
    b_store = rng.standard_normal(bb + ((n, k) if tb else (k, n)), dtype=np.float32)
    ha, hb = H.from_array(a_store), H.from_array(b_store)
    da, db = F.DeviceTensor.from_numpy(a_store), F.DeviceTensor.from_numpy(b_store)
    if ta:
        perm = tuple(range(len(ba))) + (len(ba) + 1, len(ba))
        ha, da = oracle.permute(ha, perm), da.permute(perm)
    if tb:
        perm = tuple(range(len(bb))) + (len(bb) + 1, len(bb))
        hb, db = oracle.permute(hb, perm), db.permute(perm)
    bvec = rng.standard_normal(n, dtype=np.float32) if bias else None
    if fast:
        flags |= F._lib.PRECISION_TF32
    ref = oracle.matmul(ha, hb).numpy()
    if bias:
        ref = ref + bvec
    out = F.matmul(da, db, F.DeviceTensor.from_numpy(bvec) if bias else None, flags=flags)
    F.device_status()
    tag = f"seed {seed}: ({m},{k},{n}) batches {ba}x{bb} ta={ta} tb={tb} flags={flags:#x}"
    assert out.shape == ref.shape, tag
    if fast:
        assert rel_fro(out.numpy(), ref) <= 2e-3, tag
    else:
        assert float(np.max(np.abs(out.numpy() - ref))) <= tol_3xtf32(k, a_store, b_store) + 1e-5, tag

    g = rng.standard_normal(ref.shape, dtype=np.float32)
    ga, gb = F.matmul_backward(F.DeviceTensor.from_numpy(g), da, db, flags=flags)
    F.device_status()
    ra, rb = oracle.matmul_backward(H.from_array(g), ha, hb)
    assert ga.shape == tuple(ha.shape) and gb.shape == tuple(hb.shape), tag
    if fast:
        assert rel_fro(ga.numpy(), ra.numpy()) <= 2e-3 and rel_fro(gb.numpy(), rb.numpy()) <= 2e-3, tag
    else:
        out_batch = int(np.prod(ref.shape[:-2])) if ref.ndim > 2 else 1
        fold_a = out_batch // max(int(np.prod(ba)) if ba else 1, 1)
        fold_b = out_batch // max(int(np.prod(bb)) if bb else 1, 1)
        assert float(np.max(np.abs(ga.numpy() - ra.numpy()))) <= tol_3xtf32(n * fold_a, g, b_store) + 1e-5, tag
        assert float(np.max(np.abs(gb.numpy() - rb.numpy()))) <= tol_3xtf32(m * fold_b, a_store, g) + 1e-5, tag
