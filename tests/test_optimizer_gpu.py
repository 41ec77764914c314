"""AdamW consumer of the weight gradient, gradient norm and clip_and_step against the CPU restatement of
ops/optimizer.rs:22-65, :126-138 and :226-245."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(F, a):
    return F.DeviceTensor.from_numpy(np.ascontiguousarray(a, dtype=np.float32))


def test_adamw_consumes_the_weight_gradient(F, oracle):
    """Three AdamW steps on a weight fed by matmul_backward's dW.  Both sides get the same gradient, so the
    tolerance is that of the step itself: a few ulp of the weight (fused multiply-add on the GPU, not on the CPU)."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((256, 96), dtype=np.float32)
    w = (0.02 * rng.standard_normal((96, 132))).astype(np.float32)
    cfg = dict(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1)
    w_dev = _dev(F, w)
    m_dev, v_dev = _dev(F, np.zeros_like(w)), _dev(F, np.zeros_like(w))
    w_ref, m_ref, v_ref = w.copy().ravel(), np.zeros(w.size, np.float32), np.zeros(w.size, np.float32)
    for step in (1, 2, 3):
        dy = rng.standard_normal((256, 132), dtype=np.float32)
        _, dw = F.matmul_backward(_dev(F, dy), _dev(F, x), w_dev, need_da=False)
        g = dw.numpy()
        F.adamw_step(w_dev, m_dev, v_dev, dw, step=step, **cfg)
        oracle.adamw_step(w_ref, m_ref, v_ref, g.ravel().copy(), step=step, **cfg)
        F.device_status()
        assert float(np.max(np.abs(w_dev.numpy().ravel() - w_ref))) <= 2e-6
        assert float(np.max(np.abs(m_dev.numpy().ravel() - m_ref))) <= 1e-6 * (1 + float(np.abs(g).max()))
        assert float(np.max(np.abs(v_dev.numpy().ravel() - v_ref))) <= 1e-6 * (1 + float((g * g).max()))


@pytest.mark.parametrize("n", [1, 3, 1000, 4096 * 1024 + 5])
def test_grad_norm_matches_the_f64_sum(F, oracle, n):
    """Odd sizes take the scalar tail; the f64 sum agrees with the CPU scan to f32 rounding of the result."""
    g = np.random.default_rng(n).standard_normal(n).astype(np.float32)
    got = F.grad_norm([_dev(F, g)])
    want = oracle.grad_norm([g])
    assert abs(got - want) <= 2e-7 * want


def test_grad_norm_accumulates_over_parameters(F, oracle):
    rng = np.random.default_rng(4)
    gs = [rng.standard_normal(s).astype(np.float32) for s in (7, 4096, 100_003)]
    got = F.grad_norm([_dev(F, g) for g in gs])
    want = oracle.grad_norm(gs)
    assert abs(got - want) <= 2e-7 * want
    assert F.grad_norm([]) == 0.0


@pytest.mark.parametrize("max_norm", [0.0, 1.0, 1e9])
def test_clip_and_step_matches_the_cpu_backend(F, oracle, max_norm):
    """Clip active (1.0), inactive because the norm is below it (1e9) and switched off (0): parameters,
    moments and the gradients left behind all match ops/optimizer.rs:226-245."""
    rng = np.random.default_rng(12)
    shapes = [(64, 48), (48,), (33, 5)]
    ps = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    gs = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    ms = [0.1 * rng.standard_normal(s).astype(np.float32) for s in shapes]
    vs = [np.abs(0.01 * rng.standard_normal(s)).astype(np.float32) for s in shapes]
    cfg = dict(lr=3e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, step=7, max_grad_norm=max_norm)
    dp, dm, dv, dg = ([_dev(F, a) for a in arrs] for arrs in (ps, ms, vs, gs))
    got_norm = F.clip_and_step(dp, dm, dv, dg, **cfg)
    F.device_status()
    rp, rm, rv, rg = ([a.ravel().copy() for a in arrs] for arrs in (ps, ms, vs, gs))
    want_norm = oracle.clip_and_step(rp, rm, rv, rg, **cfg)
    assert abs(got_norm - want_norm) <= 2e-7 * want_norm
    for d, r in zip(dp + dm + dv + dg, rp + rm + rv + rg):
        assert float(np.max(np.abs(d.numpy().ravel() - r))) <= 2e-6 * (1 + float(np.abs(r).max()))
    if max_norm == 1.0:
        assert oracle.grad_norm(rg) <= 1.0 + 1e-5        # the gradients left behind are the clipped ones


@pytest.mark.parametrize("step", [4, 1000, 100000, 4_000_000])
def test_adamw_bias_correction_at_large_steps(F, oracle, step):
    """ops/optimizer.rs:26-27 use f32 powi: the library must evaluate beta^step in that order (and in O(log step)
    host work).  At step 1000 with beta2 = 0.999 a sequential product gives a different bc2 and fails this bound."""
    import time
    rng = np.random.default_rng(step)
    n = 5003
    w = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    m = (0.1 * rng.standard_normal(n)).astype(np.float32)
    v = np.abs(0.01 * rng.standard_normal(n)).astype(np.float32)
    cfg = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=step)
    dw, dm, dv, dg = (_dev(F, a) for a in (w, m, v, g))
    scratch = [_dev(F, np.zeros(8, np.float32)) for _ in range(4)]
    F.adamw_step(*scratch, lr=1e-3, step=1)          # first launch of the kernel loads its module: keep that out of the timing
    F.device_status()
    t0 = time.perf_counter()
    F.adamw_step(dw, dm, dv, dg, **cfg)
    host_s = time.perf_counter() - t0
    F.device_status()
    oracle.adamw_step(w, m, v, g, **cfg)
    assert float(np.max(np.abs(dw.numpy() - w))) <= 2e-6 * (1 + float(np.abs(w).max()))
    assert host_s < 0.05, f"the call spent {host_s:.3f} s on the host"


def test_adamw_rejects_step_zero(F):
    t = _dev(F, np.zeros(8, np.float32))
    with pytest.raises(Exception):
        F.adamw_step(t, t, t, t, lr=1e-3, step=0)
