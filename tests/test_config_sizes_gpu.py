"""GPU: the benchmark configurations at their own sizes against the CPU backend (the oracle, all host
threads; its threaded form is bit-identical to the single-threaded loop).

Whole tensors where the CPU loop finishes in seconds: the Linear step (config 2), the six attention-shaped
products (config 3), the skinny products at K = N = 4096 on every route (config 5b).  The broadcast-weight
GEMM (config 4) and the 8192^3 square (config 5a) cost 0.3 - 1.1 TFLOP per product on the CPU, so there the
GPU computes the full problem and the CPU checks slices that depend only on matching slices of the inputs:
rows of C and dA need the same rows of A / dC, column panels of dB / dW need the same columns of dC (and the
whole contraction).  Bounds: max|d| <= 1e-5 * K * max|a| * max|b| (the acceptance bound) and the regression
bound on the relative Frobenius error that separates 3xTF32 from a single TF32 pass."""
import numpy as np
import pytest

from conftest import regression_bound_3xtf32, rel_fro, tol_3xtf32

pytestmark = pytest.mark.gpu


def _agree(got, ref, k, x, y, what):
    err = float(np.max(np.abs(got - ref)))
    assert err <= tol_3xtf32(k, x, y), f"{what}: max err {err:.3e}"
    r = rel_fro(got, ref)
    assert r <= regression_bound_3xtf32(k), f"{what}: relative Frobenius error {r:.2e} (K = {k})"


def test_config2_linear_step_full_size(F, oracle):
    """x[4096,1024] ~U[0,1) . W[1024,4096] ~N(0,0.02) + b, dy ~N(0,1): y, dx, dW, db; bias zeros and N(0,0.02)."""
    rng = np.random.default_rng(0)
    x = rng.random((4096, 1024), dtype=np.float32)
    w = (0.02 * rng.standard_normal((1024, 4096))).astype(np.float32)
    dy = rng.standard_normal((4096, 4096), dtype=np.float32)
    H, t = oracle.HostTensor, F.DeviceTensor.from_numpy
    hx, hw, hdy = H.from_array(x), H.from_array(w), H.from_array(dy)
    xw = oracle.matmul(hx, hw)
    xd, wd, dyd = t(x), t(w), t(dy)
    for bias in (np.zeros(4096, np.float32), (0.02 * rng.standard_normal(4096)).astype(np.float32)):
        ref = oracle.add(xw, H.from_array(bias)).numpy()
        _agree(F.matmul(xd, wd, t(bias)).numpy(), ref, 1024, x, w, "y (fused bias)")
        _agree(F.Linear(wd, t(bias)).forward(xd).numpy(), ref, 1024, x, w, "y (matmul, then add)")
    rdx, rdw = oracle.matmul_backward(hdy, hx, hw)
    _, rdb = oracle.add_backward(hdy, hdy.shape, (4096,))
    dx, dw, db = F.matmul_backward(dyd, xd, wd, want_dbias=True)
    F.device_status()
    _agree(dx.numpy(), rdx.numpy(), 4096, dy, w, "dx")
    _agree(dw.numpy(), rdw.numpy(), 4096, x, dy, "dW")
    assert float(np.max(np.abs(db.numpy() - rdb.numpy()))) <= 1e-5 * 4096 * float(np.abs(dy).max())
    assert rel_fro(db.numpy(), rdb.numpy()) <= 1e-5


def test_config3_attention_shaped_full_size(F, oracle):
    """Q,K,V [8,12,512,64] ~N(0,1): S = Q.K^T through the permute(0,1,3,2) view, O = S.V, backward from dO ~N(0,1):
    all six products, dK returned in K's layout."""
    rng = np.random.default_rng(0)
    q, k, v, do = (rng.standard_normal((8, 12, 512, 64), dtype=np.float32) for _ in range(4))
    H, t = oracle.HostTensor, F.DeviceTensor.from_numpy
    hq, hv, hdo = H.from_array(q), H.from_array(v), H.from_array(do)
    hkt = oracle.permute(H.from_array(k), [0, 1, 3, 2])
    rs = oracle.matmul(hq, hkt)
    ro = oracle.matmul(rs, hv)
    rds, rdv = oracle.matmul_backward(hdo, rs, hv)
    rdq, rdkt = oracle.matmul_backward(rds, hq, hkt)
    rdk = oracle.permute_backward(rdkt, [0, 1, 3, 2], k.shape)
    qd, vd, dod = t(q), t(v), t(do)
    ktd = t(k).permute([0, 1, 3, 2])
    assert not ktd.is_contiguous() and ktd.strides == (393216, 32768, 1, 64)
    s = F.matmul(qd, ktd)
    o = F.matmul(s, vd)
    ds, dv = F.matmul_backward(dod, s, vd)
    dq, dkt = F.matmul_backward(ds, qd, ktd)
    dk = F.permute_backward(dkt, [0, 1, 3, 2], k.shape)
    F.device_status()
    sn, dsn = rs.numpy(), rds.numpy()
    _agree(s.numpy(), sn, 64, q, k, "S")
    _agree(o.numpy(), ro.numpy(), 512, sn, v, "O")
    _agree(ds.numpy(), dsn, 64, do, v, "dS")
    _agree(dv.numpy(), rdv.numpy(), 512, sn, do, "dV")
    _agree(dq.numpy(), rdq.numpy(), 512, dsn, k, "dQ")
    _agree(dk.numpy(), rdk.numpy(), 512, q, dsn, "dK")


@pytest.mark.parametrize("m", [1, 4, 16])
@pytest.mark.parametrize("route", ["default", "skinny", "tensor"])
def test_config5b_skinny_full_size(F, oracle, m, route):
    """x[M,4096] . W[4096,4096] ~N(0,1), dy ~N(0,1): y, dx, dW on the route the library picks, forced onto the
    streaming kernels and forced onto the tensor cores (where the 8-way split / cluster plans of this size run)."""
    flags = {"default": 0, "skinny": F._lib.FORCE_SKINNY_PATH, "tensor": F._lib.FORCE_TENSOR_PATH}[route]
    rng = np.random.default_rng(m)
    x = rng.standard_normal((m, 4096), dtype=np.float32)
    w = rng.standard_normal((4096, 4096), dtype=np.float32)
    dy = rng.standard_normal((m, 4096), dtype=np.float32)
    H, t = oracle.HostTensor, F.DeviceTensor.from_numpy
    ry = oracle.matmul(H.from_array(x), H.from_array(w)).numpy()
    rdx, rdw = oracle.matmul_backward(H.from_array(dy), H.from_array(x), H.from_array(w))
    y = F.matmul(t(x), t(w), flags=flags)
    dx, dw = F.matmul_backward(t(dy), t(x), t(w), flags=flags)
    F.device_status()
    _agree(y.numpy(), ry, 4096, x, w, f"y M={m} {route}")
    _agree(dx.numpy(), rdx.numpy(), 4096, dy, w, f"dx M={m} {route}")
    _agree(dw.numpy(), rdw.numpy(), m, x, dy, f"dW M={m} {route}")


def _row_slices(rows, step=128):
    return [slice(0, step), slice(rows - step, rows)]


def test_config4_broadcast_weight_full_size_slices(F, oracle):
    """A[64,1024,768] ~N(0,1) . W[768,3072] ~N(0,0.02), dC ~N(0,1): the GPU runs the full problem; the CPU checks
    the first 128 rows of batch 0 and the last 128 rows of batch 63 of C and dA, and two 128-column panels of dW
    with the contraction over all 64 x 1024 rows, in the reference's order (per-batch products, then the
    unbroadcast sum over batches, ops/matmul.rs:242-251, utils.rs:39-66)."""
    rng = np.random.default_rng(0)
    a = rng.standard_normal((64, 1024, 768), dtype=np.float32)
    w = (0.02 * rng.standard_normal((768, 3072))).astype(np.float32)
    dc = rng.standard_normal((64, 1024, 3072), dtype=np.float32)
    H, t = oracle.HostTensor, F.DeviceTensor.from_numpy
    ad, wd, dcd = t(a), t(w), t(dc)
    c = F.matmul(ad, wd).numpy()
    da, dw = (x.numpy() for x in F.matmul_backward(dcd, ad, wd))
    F.device_status()
    hw = H.from_array(w)
    hwt = oracle.permute(hw, [1, 0])
    for bt, rows in ((0, slice(0, 128)), (63, slice(896, 1024))):
        ref_c = oracle.matmul(H.from_array(a[bt, rows]), hw).numpy()
        _agree(c[bt, rows], ref_c, 768, a, w, f"C batch {bt}")
        ref_da = oracle.matmul(H.from_array(dc[bt, rows]), hwt).numpy()        # dC . W^T, ops/matmul.rs:231-232
        _agree(da[bt, rows], ref_da, 3072, dc, w, f"dA batch {bt}")
    for cols in (slice(0, 128), slice(2944, 3072)):
        panel = np.ascontiguousarray(dc[:, :, cols])
        _, ref_dw = oracle.matmul_backward(H.from_array(panel), H.from_array(a), H.from_array(w[:, cols]))
        _agree(dw[:, cols], ref_dw.numpy(), 64 * 1024, a, dc, f"dW columns {cols.start}")


def test_config5a_square_8192_full_size_slices(F, oracle):
    """A, B, dC [8192,8192] ~N(0,1): first and last 128 rows of C and dA, two 128-column panels of dB."""
    rng = np.random.default_rng(0)
    a = rng.standard_normal((8192, 8192), dtype=np.float32)
    b = rng.standard_normal((8192, 8192), dtype=np.float32)
    dc = rng.standard_normal((8192, 8192), dtype=np.float32)
    H, t = oracle.HostTensor, F.DeviceTensor.from_numpy
    ad, bd, dcd = t(a), t(b), t(dc)
    c = F.matmul(ad, bd).numpy()
    da, db = (x.numpy() for x in F.matmul_backward(dcd, ad, bd))
    F.device_status()
    hb = H.from_array(b)
    hbt = oracle.permute(hb, [1, 0])
    for rows in _row_slices(8192):
        _agree(c[rows], oracle.matmul(H.from_array(a[rows]), hb).numpy(), 8192, a, b, f"C rows {rows.start}")
        _agree(da[rows], oracle.matmul(H.from_array(dc[rows]), hbt).numpy(), 8192, dc, b, f"dA rows {rows.start}")
    hat = oracle.permute(H.from_array(a), [1, 0])
    for cols in (slice(0, 128), slice(8064, 8192)):
        ref = oracle.matmul(hat, H.from_array(np.ascontiguousarray(dc[:, cols]))).numpy()   # A^T . dC, :242-243
        _agree(db[:, cols], ref, 8192, a, dc, f"dB columns {cols.start}")
