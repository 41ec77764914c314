"""GPU: whole-tensor checks at the full sizes of the benchmark configurations, where the CPU oracle only
covers slices (tests/test_config_sizes_gpu.py).  Freivalds' identity: for C = A.B and a random vector v,
C.v == A.(B.v); the right side costs two matrix-vector products in float64.  With v ~N(0,1) and every
element of C within e = 1e-5 * K * max|a| * max|b| of the truth, a row of (C - AB).v has a standard
deviation of at most e * sqrt(N); the test allows 4 of them (the maximum over thousands of rows), not the
e * sum|v| a worst-case alignment of signs would give."""
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


def _freivalds(c, a, b, k):
    """c, a, b: torch tensors [..., M, N], [..., M, K], [..., K, N] (broadcastable batches)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(7)
    v = torch.randn(c.shape[-1], 1, device="cuda", dtype=torch.float64, generator=g)
    left = c.double() @ v
    right = a.double() @ (b.double() @ v)
    bound = 1e-5 * k * float(a.abs().max()) * float(b.abs().max()) * 4.0 * float(c.shape[-1]) ** 0.5
    return float((left - right).abs().max()), bound


def test_square_8192_forward_and_backward(F):
    import torch
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn(8192, 8192, device="cuda", generator=g)
    b = torch.randn(8192, 8192, device="cuda", generator=g)
    dc = torch.randn(8192, 8192, device="cuda", generator=g)
    t = F.DeviceTensor.from_torch
    c = F.matmul(t(a), t(b)).torch_view()
    da, db = F.matmul_backward(t(dc), t(a), t(b))
    F.device_status()
    for got, x, y in ((c, a, b), (da.torch_view(), dc, b.t()), (db.torch_view(), a.t(), dc)):
        err, bound = _freivalds(got, x, y, 8192)
        assert err <= bound, (err, bound)


def test_broadcast_weight_full_size(F):
    """[64,1024,768] . [768,3072]; dW = sum over the 64 batches (contraction 65536 long)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(64, 1024, 768, device="cuda", generator=g)
    w = 0.02 * torch.randn(768, 3072, device="cuda", generator=g)
    dc = torch.randn(64, 1024, 3072, device="cuda", generator=g)
    t = F.DeviceTensor.from_torch
    c = F.matmul(t(a), t(w)).torch_view()
    da, dw = F.matmul_backward(t(dc), t(a), t(w))
    F.device_status()
    err, bound = _freivalds(c, a, w, 768)
    assert err <= bound
    err, bound = _freivalds(da.torch_view(), dc, w.t(), 3072)
    assert err <= bound
    a2, dc2 = a.reshape(-1, 768), dc.reshape(-1, 3072)
    err, bound = _freivalds(dw.torch_view(), a2.t(), dc2, 65536)
    assert err <= bound


def test_attention_shaped_full_size(F):
    """Q,K,V [8,12,512,64]; K^T read as a permute view; all six products."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(2)
    q, k, v, do = (torch.randn(8, 12, 512, 64, device="cuda", generator=g) for _ in range(4))
    t = F.DeviceTensor.from_torch
    kt = t(k).permute([0, 1, 3, 2])
    s = F.matmul(t(q), kt)
    o = F.matmul(s, t(v))
    ds, dv = F.matmul_backward(t(do), s, t(v))
    dq, dkt = F.matmul_backward(ds, t(q), kt)
    F.device_status()
    S, dS = s.torch_view(), ds.torch_view()
    checks = [(S, q, k.transpose(-1, -2), 64), (o.torch_view(), S, v, 512), (dS, do, v.transpose(-1, -2), 64),
              (dv.torch_view(), S.transpose(-1, -2), do, 512), (dq.torch_view(), dS, k, 512),
              (dkt.torch_view(), q.transpose(-1, -2), dS, 512)]
    for got, x, y, kk in checks:
        err, bound = _freivalds(got, x, y, kk)
        assert err <= bound, (err, bound)


def test_caller_provided_workspace(F):
    """mni_b200_workspace_query / _set: the library must run inside the caller's scratch and refuse one
    that is too small instead of allocating."""
    import ctypes as C
    import torch
    lib = F._lib.lib()
    rng = np.random.default_rng(3)
    a = F.DeviceTensor.from_numpy(rng.standard_normal((6, 96, 50), dtype=np.float32))     # K = 50: packed fallback
    w = F.DeviceTensor.from_numpy(rng.standard_normal((50, 72), dtype=np.float32))
    dc = F.DeviceTensor.from_numpy(rng.standard_normal((6, 96, 72), dtype=np.float32))
    ref_c = F.matmul(a, w).numpy()
    ref_da, ref_dw = (x.numpy() for x in F.matmul_backward(dc, a, w))
    need = C.c_size_t(0)
    va, vw = a.view_struct(), w.view_struct()
    F._lib.check(lib.mni_b200_workspace_query(va, vw, 0, C.byref(need)))
    assert need.value > 0
    # the caller's buffer sits between two canary zones: the library must stay inside the bytes it was given
    guard, canary = 4096, 0x5A
    buf = torch.full((need.value + 2 * guard + 256,), canary, dtype=torch.uint8, device="cuda")
    base = (buf.data_ptr() + guard + 255) // 256 * 256
    lo = base - buf.data_ptr()
    try:
        F._lib.check(lib.mni_b200_workspace_set(C.c_void_p(base), need.value))
        assert np.array_equal(F.matmul(a, w).numpy(), ref_c)
        da, dw = F.matmul_backward(dc, a, w)
        assert np.array_equal(da.numpy(), ref_da) and np.array_equal(dw.numpy(), ref_dw)
        torch.cuda.synchronize()
        assert bool((buf[:lo] == canary).all()) and bool((buf[lo + need.value:] == canary).all()), \
            "the library wrote outside the caller-provided scratch"
        assert not bool((buf[lo:lo + need.value] == canary).all()), "the caller-provided scratch was never used"
        F._lib.check(lib.mni_b200_workspace_set(C.c_void_p(base), 256))
        with pytest.raises(F._lib.MniError) as ei:
            F.matmul_backward(dc, a, w)
        assert ei.value.status == 7
    finally:
        F._lib.check(lib.mni_b200_workspace_set(None, 0))
    assert np.array_equal(F.matmul(a, w).numpy(), ref_c)
