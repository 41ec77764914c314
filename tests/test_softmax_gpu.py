"""Softmax forward/backward (the step between the two attention GEMMs) against the CPU restatement of
ops/norm.rs:10-50 and :95-123.  Tolerance: the GPU's expf and the CPU's differ by an ulp or two and the sums
run in another order, so |delta| <= 4e-7 + 4e-6 * |ref| for the forward (outputs lie in [0, 1])."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(F, a):
    return F.DeviceTensor.from_numpy(np.ascontiguousarray(a, dtype=np.float32))


def _close(got, want, atol, rtol):
    assert got.shape == want.shape
    assert np.all(np.abs(got - want) <= atol + rtol * np.abs(want)), float(np.max(np.abs(got - want)))


SHAPES = [
    ((2, 3), 1),                 # the reference's own test case
    ((2, 3), 0),
    ((5, 1), -1),                # length-1 rows: all ones
    ((64, 128), -1),             # one float4 chunk per lane
    ((33, 516), -1),             # ragged last chunk
    ((2, 3, 512, 512), -1),      # attention-shaped rows
    ((7, 2048), -1),             # the longest row kept in registers
    ((3, 4100), -1),             # longer: block per row
    ((9, 130), -1),              # length not a multiple of 4: block per row
    ((4, 96, 40), 1),            # softmax over a middle dimension
    ((50, 7), 0),
]


@pytest.mark.parametrize("shape,dim", SHAPES)
def test_softmax_forward_and_backward(F, oracle, shape, dim):
    rng = np.random.default_rng(abs(hash((shape, dim))) % (2 ** 31))
    x = (3.0 * rng.standard_normal(shape)).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    sm_ref = oracle.softmax(x, dim)
    sm = F.softmax(_dev(F, x), dim)
    F.device_status()
    _close(sm.numpy(), sm_ref, 4e-7, 4e-6)
    # backward from the same saved output on both sides
    dx_ref = oracle.softmax_backward(g, sm_ref, dim)
    dx = F.softmax_backward(_dev(F, g), _dev(F, sm_ref), dim)
    F.device_status()
    _close(dx.numpy(), dx_ref, 2e-6, 1e-5)


def test_softmax_of_a_permuted_view(F, oracle):
    """A strided input is gathered on the device first; the result is that of the logical tensor."""
    x = np.random.default_rng(1).standard_normal((6, 40, 24)).astype(np.float32)
    xt = _dev(F, x).permute((0, 2, 1))
    sm = F.softmax(xt, -1)
    _close(sm.numpy(), oracle.softmax(np.transpose(x, (0, 2, 1)), -1), 4e-7, 4e-6)


def test_softmax_handles_large_magnitudes_and_empty(F, oracle):
    x = np.array([[1e4, 1e4 - 1, -1e4, 0.0], [-3e38, -3e38, -3e38, -3e38]], np.float32)
    _close(F.softmax(_dev(F, x), -1).numpy(), oracle.softmax(x, -1), 4e-7, 4e-6)
    empty = F.DeviceTensor.empty((0, 8))
    assert F.softmax(empty, -1).shape == (0, 8)


def test_attention_block_through_the_path(F, oracle):
    """S = Q.K^T (K permuted, no copy) -> softmax -> O = P.V and the whole backward, against the oracle chain."""
    rng = np.random.default_rng(5)
    B, H, T, D = 2, 3, 128, 64
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    q *= 0.125
    do = rng.standard_normal((B, H, T, D)).astype(np.float32)
    qd, kd, vd = _dev(F, q), _dev(F, k), _dev(F, v)
    kt = kd.permute((0, 1, 3, 2))
    s = F.matmul(qd, kt)
    p = F.softmax(s, -1)
    o = F.matmul(p, vd)
    dp, dv = F.matmul_backward(_dev(F, do), p, vd)
    ds = F.softmax_backward(dp, p, -1)
    dq, dkt = F.matmul_backward(ds, qd, kt)
    F.device_status()

    H_ = oracle.HostTensor
    s_ref = oracle.matmul(H_.from_array(q), oracle.permute(H_.from_array(k), (0, 1, 3, 2))).numpy()
    p_ref = oracle.softmax(s_ref, -1)
    o_ref = oracle.matmul(H_.from_array(p_ref), H_.from_array(v)).numpy()
    dp_ref, dv_ref = oracle.matmul_backward(H_.from_array(do), H_.from_array(p_ref), H_.from_array(v))
    ds_ref = oracle.softmax_backward(dp_ref.numpy(), p_ref, -1)
    dq_ref, dkt_ref = oracle.matmul_backward(H_.from_array(ds_ref), H_.from_array(q),
                                             oracle.permute(H_.from_array(k), (0, 1, 3, 2)))
    tol = lambda kk, a, b: 1e-5 * kk * float(np.abs(a).max()) * float(np.abs(b).max())
    assert np.max(np.abs(o.numpy() - o_ref)) <= tol(T, p_ref, v) + 1e-5
    assert np.max(np.abs(dv.numpy() - dv_ref.numpy())) <= tol(T, p_ref, do) + 1e-5
    assert np.max(np.abs(dq.numpy() - dq_ref.numpy())) <= tol(T, ds_ref, k) + 1e-5
    assert np.max(np.abs(dkt.numpy() - dkt_ref.numpy())) <= tol(T, ds_ref, q) + 1e-5
