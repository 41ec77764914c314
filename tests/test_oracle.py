"""CPU: the oracle against the reference's own known answers and against independent maths."""
import numpy as np
import pytest


def _t(O, shape, data):
    return O.HostTensor.from_array(np.array(data, np.float32).reshape(shape))


def test_reference_forward_known_answers(oracle, golden):
    O = oracle
    for case in golden["forward"]:
        out = O.matmul(_t(O, **case["a"]), _t(O, **case["b"]), threads=1)
        assert list(out.shape) == case["out"]["shape"], case["source"]
        if "data" in case["out"]:
            np.testing.assert_allclose(out.data, case["out"]["data"], atol=case["tol"])
        else:
            assert abs(out.data[0] - case["out"]["first"]) <= case["tol"]


def test_reference_forward_shapes(oracle, golden):
    O = oracle
    rng = np.random.default_rng(1)
    for case in golden["forward_shapes"]:
        a = O.HostTensor.from_array(rng.random(case["a"], dtype=np.float32))
        b = O.HostTensor.from_array(rng.random(case["b"], dtype=np.float32))
        out = O.matmul(a, b)
        if "bias" in case:
            out = O.add(out, O.HostTensor.from_array(rng.random(case["bias"], dtype=np.float32)))
        assert list(out.shape) == case["out"], case["source"]


def test_reference_backward_known_answers(oracle, golden):
    O = oracle
    for case in golden["backward"]:
        da, db = O.matmul_backward(_t(O, **case["grad"]), _t(O, **case["a"]), _t(O, **case["b"]), threads=1)
        np.testing.assert_array_equal(da.data, np.array(case["da"], np.float32))
        np.testing.assert_array_equal(db.data, np.array(case["db"], np.float32))


@pytest.mark.parametrize("shape_a,shape_b", [((64, 48), (48, 40)), ((3, 17, 9), (3, 9, 11)),
                                             ((5, 8, 16), (16, 12)), ((7, 6), (2, 6, 5))])
def test_threads_are_bit_identical(oracle, shape_a, shape_b):
    O = oracle
    rng = np.random.default_rng(2)
    a = O.HostTensor.from_array(rng.standard_normal(shape_a, dtype=np.float32))
    b = O.HostTensor.from_array(rng.standard_normal(shape_b, dtype=np.float32))
    c1 = O.matmul(a, b, threads=1)
    c4 = O.matmul(a, b, threads=4)
    assert np.array_equal(c1.data, c4.data)
    g = O.HostTensor.from_array(rng.standard_normal(c1.shape, dtype=np.float32))
    da1, db1 = O.matmul_backward(g, a, b, threads=1)
    da4, db4 = O.matmul_backward(g, a, b, threads=4)
    assert np.array_equal(da1.data, da4.data) and np.array_equal(db1.data, db4.data)


def test_loop_order_is_k_ascending_without_fma(oracle):
    """One output element must equal the sequential f32 mul-then-add chain of ops/matmul.rs:62-68."""
    O = oracle
    rng = np.random.default_rng(3)
    a = rng.standard_normal((4, 300), dtype=np.float32)
    b = rng.standard_normal((300, 5), dtype=np.float32)
    out = O.matmul(O.HostTensor.from_array(a), O.HostTensor.from_array(b), threads=1).data.reshape(4, 5)
    for i, j in [(0, 0), (3, 4), (2, 1)]:
        acc = np.float32(0.0)
        for k in range(300):
            acc = np.float32(acc + np.float32(a[i, k] * b[k, j]))
        assert out[i, j] == acc


def test_matches_float64_closely(oracle):
    O = oracle
    rng = np.random.default_rng(4)
    a = rng.standard_normal((6, 33, 70), dtype=np.float32)
    b = rng.standard_normal((70, 21), dtype=np.float32)
    out = O.matmul(O.HostTensor.from_array(a), O.HostTensor.from_array(b)).numpy()
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert np.max(np.abs(out - ref)) < 1e-4
    g = rng.standard_normal(out.shape, dtype=np.float32)
    da, db = O.matmul_backward(O.HostTensor.from_array(g), O.HostTensor.from_array(a), O.HostTensor.from_array(b))
    np.testing.assert_allclose(da.numpy(), g.astype(np.float64) @ b.T.astype(np.float64), atol=2e-4)
    dbr = np.einsum("bmk,bmn->kn", a.astype(np.float64), g.astype(np.float64))
    np.testing.assert_allclose(db.numpy(), dbr, atol=1e-3)


def test_strided_views_are_gathered(oracle):
    """permute gives a stride-only view (ops/layout.rs:112-134); matmul reads it through ensure_contiguous."""
    O = oracle
    rng = np.random.default_rng(5)
    q = rng.standard_normal((2, 3, 8, 4), dtype=np.float32)
    k = rng.standard_normal((2, 3, 8, 4), dtype=np.float32)
    kt = O.permute(O.HostTensor.from_array(k), [0, 1, 3, 2])
    assert kt.shape == (2, 3, 4, 8) and kt.strides == (96, 32, 1, 4) and not kt.is_contiguous()
    s = O.matmul(O.HostTensor.from_array(q), kt).numpy()
    np.testing.assert_allclose(s, q @ np.swapaxes(k, -1, -2), atol=1e-5)
    g = O.HostTensor.from_array(np.ones((2, 3, 4, 8), np.float32))
    back = O.permute_backward(g, [0, 1, 3, 2], (2, 3, 8, 4))
    assert back.shape == (2, 3, 8, 4)


def test_non_simple_broadcast_uses_modulo_indexing(oracle):
    """ops/matmul.rs:55-56: operand batch index is `batch % operand_batch`, not true N-D broadcasting."""
    O = oracle
    rng = np.random.default_rng(6)
    a = rng.standard_normal((2, 1, 3, 4), dtype=np.float32)
    b = rng.standard_normal((1, 3, 4, 5), dtype=np.float32)
    out = O.matmul(O.HostTensor.from_array(a), O.HostTensor.from_array(b)).numpy()
    assert out.shape == (2, 3, 3, 5)
    flat = out.reshape(6, 3, 5)
    for batch in range(6):
        np.testing.assert_allclose(flat[batch], a.reshape(2, 3, 4)[batch % 2] @ b.reshape(3, 4, 5)[batch % 3],
                                   atol=1e-5)


def test_unbroadcast_backward_of_shared_weight(oracle):
    O = oracle
    rng = np.random.default_rng(7)
    a = rng.standard_normal((5, 6, 7), dtype=np.float32)
    w = rng.standard_normal((7, 3), dtype=np.float32)
    g = rng.standard_normal((5, 6, 3), dtype=np.float32)
    da, dw = O.matmul_backward(O.HostTensor.from_array(g), O.HostTensor.from_array(a), O.HostTensor.from_array(w),
                               threads=1)
    assert da.shape == (5, 6, 7) and dw.shape == (7, 3)
    # two-level order of the reference: per-batch products, then batches added in ascending order
    per = np.stack([a[i].T.astype(np.float64) @ g[i].astype(np.float64) for i in range(5)])
    np.testing.assert_allclose(dw.numpy(), per.sum(0), atol=1e-4)


def test_bias_add_and_backward(oracle):
    O = oracle
    rng = np.random.default_rng(8)
    y = rng.standard_normal((4, 6), dtype=np.float32)
    bias = rng.standard_normal((6,), dtype=np.float32)
    out = O.add(O.HostTensor.from_array(y), O.HostTensor.from_array(bias))
    assert np.array_equal(out.numpy(), y + bias)
    g = rng.standard_normal((4, 6), dtype=np.float32)
    ga, gb = O.add_backward(O.HostTensor.from_array(g), (4, 6), (6,), threads=1)
    assert np.array_equal(ga.numpy(), g)
    acc = np.zeros(6, np.float32)
    for r in range(4):
        acc = (acc + g[r]).astype(np.float32)
    assert np.array_equal(gb.numpy(), acc)


def test_error_cases(oracle):
    O = oracle
    a = O.HostTensor.from_array(np.zeros((2, 3), np.float32))
    with pytest.raises(ValueError, match="inner dimensions"):
        O.matmul(a, O.HostTensor.from_array(np.zeros((4, 2), np.float32)))
    with pytest.raises(ValueError, match="at least 2D"):
        O.matmul(a, O.HostTensor.from_array(np.zeros((3,), np.float32)))
    with pytest.raises(ValueError, match="broadcastable"):
        O.matmul(O.HostTensor.from_array(np.zeros((2, 2, 3), np.float32)),
                 O.HostTensor.from_array(np.zeros((3, 3, 2), np.float32)))


def test_adamw_first_step_moves_by_lr_times_sign(oracle):
    """ops/optimizer.rs:22-65: with zero moments, step 1 gives m_hat = g and v_hat = g*g, so every weight moves
    by lr * g / (|g| + eps) after the decoupled decay; checked against float64 arithmetic of the same formula."""
    rng = np.random.default_rng(0)
    w = rng.standard_normal(1001).astype(np.float32)
    g = rng.standard_normal(1001).astype(np.float32)
    m, v = np.zeros_like(w), np.zeros_like(w)
    w0 = w.copy()
    oracle.adamw_step(w, m, v, g, lr=1e-2, weight_decay=0.1, step=1)
    g64 = g.astype(np.float64)
    want = w0.astype(np.float64) * (1 - 1e-2 * 0.1) - 1e-2 * g64 / (np.abs(g64) + 1e-8)
    assert np.max(np.abs(w - want)) < 1e-6
    assert np.allclose(m, 0.1 * g, rtol=1e-6) and np.allclose(v, 0.001 * g * g, rtol=1e-4)  # 1 - 0.999f is 0.00100005
    # a second step with zero gradient only decays the moments
    oracle.adamw_step(w, m, v, np.zeros_like(g), lr=0.0, step=2)
    assert np.allclose(m, 0.09 * g, rtol=1e-6)


def _powi_f32(x, n):
    """Independent restatement of f32::powi (binary exponentiation, lowest bit first) in numpy float32."""
    x, r = np.float32(x), np.float32(1.0)
    while True:
        if n & 1:
            r = np.float32(r * x)
        n >>= 1
        if n == 0:
            return float(r)
        x = np.float32(x * x)


def test_bias_correction_uses_powi_rounding(oracle):
    """ops/optimizer.rs:26-27: bc = 1 - beta.powi(step).  powi squares repeatedly, so from step 4 on it rounds
    differently from `step` successive multiplications; large steps must follow powi, in O(log step)."""
    for beta in (0.9, 0.95, 0.999):
        for step in (1, 2, 3, 4, 7, 1000, 100000):
            assert oracle.powi(beta, step) == _powi_f32(beta, step), (beta, step)
    # hand-derived: 0.5^10 is exact, 2^-20 too; a negative exponent takes the reciprocal
    assert oracle.powi(0.5, 10) == 2.0 ** -10 and oracle.powi(2.0, -20) == 2.0 ** -20
    # the two evaluation orders do differ in f32 (this is what the parity case at step 1000 guards)
    seq = np.float32(1.0)
    for _ in range(1000):
        seq = np.float32(seq * np.float32(0.999))
    assert float(seq) != oracle.powi(0.999, 1000)
    # and the step itself follows: one AdamW step at step = 1000 against the formula in float64 with powi's bc
    rng = np.random.default_rng(5)
    w, g = rng.standard_normal(257).astype(np.float32), rng.standard_normal(257).astype(np.float32)
    m, v = (0.1 * rng.standard_normal(257)).astype(np.float32), np.abs(0.01 * rng.standard_normal(257)).astype(np.float32)
    w0, m0, v0 = w.copy(), m.copy(), v.copy()
    oracle.adamw_step(w, m, v, g, lr=1e-3, beta1=0.9, beta2=0.999, step=1000)
    bc1 = 1.0 - _powi_f32(0.9, 1000)
    bc2 = np.float32(1.0) - np.float32(_powi_f32(0.999, 1000))
    m1 = np.float32(0.9) * m0 + (np.float32(1.0) - np.float32(0.9)) * g
    v1 = np.float32(0.999) * v0 + (np.float32(1.0) - np.float32(0.999)) * g * g
    want = w0.astype(np.float64) - 1e-3 * (m1.astype(np.float64) / bc1) / (np.sqrt(v1.astype(np.float64) / float(bc2)) + 1e-8)
    assert np.max(np.abs(w - want)) < 2e-6


def test_clip_and_step_scales_the_gradients_in_place(oracle):
    """ops/optimizer.rs:226-245: the norm is returned unclipped, the gradients are left scaled to max_grad_norm."""
    g = [np.full(4, 3.0, np.float32), np.full(9, 4.0, np.float32)]       # norm = sqrt(36 + 144)
    p = [np.ones(4, np.float32), np.ones(9, np.float32)]
    m = [np.zeros(4, np.float32), np.zeros(9, np.float32)]
    v = [np.zeros(4, np.float32), np.zeros(9, np.float32)]
    assert abs(oracle.grad_norm(g) - np.sqrt(180.0)) < 1e-5
    norm = oracle.clip_and_step(p, m, v, g, lr=0.1, step=1, max_grad_norm=1.0)
    assert abs(norm - np.sqrt(180.0)) < 1e-5
    assert abs(oracle.grad_norm(g) - 1.0) < 1e-6
    assert np.allclose(p[0], 0.9, atol=1e-6) and np.allclose(p[1], 0.9, atol=1e-6)   # lr * sign(g)


def test_softmax_reference_checks(oracle):
    """The reference's own softmax checks (test/nn.test.ts:47-54): input [[1,2,3],[1,2,3]], dim 1 — rows sum to 1
    within 1e-4, all positive, ordering preserved; plus the closed form and the backward's zero row sums."""
    x = np.array([[1, 2, 3], [1, 2, 3]], np.float32)
    sm = oracle.softmax(x, 1)
    assert abs(sm[0].sum() - 1.0) < 1e-4 and abs(sm[1].sum() - 1.0) < 1e-4
    assert (sm > 0).all() and sm[0, 2] > sm[0, 1] > sm[0, 0]
    want = np.exp(x.astype(np.float64) - 3.0)
    want /= want.sum(axis=1, keepdims=True)
    assert np.max(np.abs(sm - want)) < 1e-7
    # over dim 0 both entries of a column are equal
    assert np.allclose(oracle.softmax(x, 0), 0.5)
    g = np.array([[0.5, -1.0, 2.0], [1.0, 1.0, 1.0]], np.float32)
    dx = oracle.softmax_backward(g, sm, 1)
    assert np.max(np.abs(dx.sum(axis=1))) < 1e-6          # softmax gradients sum to zero along the dim
    assert np.max(np.abs(dx[1])) < 1e-7                   # a constant upstream gradient gives zero
    j = np.diag(want[0]) - np.outer(want[0], want[0])     # Jacobian of softmax
    assert np.max(np.abs(dx[0] - j @ g[0].astype(np.float64))) < 1e-6


def _numeric_grad(f, x, eps=1e-3):
    """Central differences of the scalar f with respect to every element of x (float64)."""
    g = np.zeros_like(x, dtype=np.float64)
    flat, gf = x.reshape(-1), g.reshape(-1)
    for i in range(flat.size):
        keep = flat[i]
        flat[i] = keep + eps
        hi = f()
        flat[i] = keep - eps
        lo = f()
        flat[i] = keep
        gf[i] = (hi - lo) / (2 * eps)
    return g


@pytest.mark.parametrize("shape_a,shape_b", [
    ((3, 4), (4, 2)),                  # 2-D
    ((2, 3, 4), (2, 4, 5)),            # batched
    ((3, 2, 4), (4, 5)),               # weight shared by every batch: grad_b is summed over the batches
    ((2, 3, 3, 4), (1, 3, 4, 2)),      # b broadcast along the leading batch dim (batch % 3 = true broadcasting here)
])
def test_backward_is_the_derivative_of_the_forward(oracle, shape_a, shape_b):
    """The reference's tests hold no backward values (test/autograd.test.ts:41-46 only asks that a gradient
    exists), so the backward restatement is pinned here by what it must be: the derivative of
    loss = sum(grad * forward(a, b)), taken by central differences in float64 through NumPy's own broadcasting
    matmul -- a computation that shares nothing with ops/matmul.rs:200-222 (transposes, products, unbroadcast).
    Shapes where each operand broadcasts along a different batch dim are left out on purpose: there the
    reference's forward indexes `batch % operand_batch` (ops/matmul.rs:55-56) while its backward un-broadcasts
    by position (utils.rs:39-66), so its own backward is not the derivative of its own forward; the oracle
    follows the reference in both (test_non_simple_broadcast_uses_modulo_indexing)."""
    O = oracle
    rng = np.random.default_rng(11)
    a = rng.standard_normal(shape_a)
    b = rng.standard_normal(shape_b)
    g = rng.standard_normal(np.matmul(a, b).shape)
    loss = lambda: float(np.sum(g * np.matmul(a, b)))   # noqa: E731
    na, nb = _numeric_grad(loss, a), _numeric_grad(loss, b)
    H = O.HostTensor
    da, db = O.matmul_backward(H.from_array(g.astype(np.float32)), H.from_array(a.astype(np.float32)),
                               H.from_array(b.astype(np.float32)), threads=1)
    assert da.shape == shape_a and db.shape == shape_b
    np.testing.assert_allclose(da.numpy(), na, rtol=2e-4, atol=2e-4)
    np.testing.assert_allclose(db.numpy(), nb, rtol=2e-4, atol=2e-4)


def test_permuted_operand_backward_is_the_derivative(oracle):
    """S = Q . K^T with K^T a stride-only permute of K (the attention-shaped configuration): the gradient that
    reaches K through permute_backward (ops/layout.rs:162-195) is the derivative with respect to K's storage."""
    O = oracle
    rng = np.random.default_rng(12)
    q = rng.standard_normal((2, 3, 4))
    k = rng.standard_normal((2, 5, 4))
    g = rng.standard_normal((2, 3, 5))
    loss = lambda: float(np.sum(g * np.matmul(q, np.swapaxes(k, 1, 2))))   # noqa: E731
    nk = _numeric_grad(loss, k)
    H = O.HostTensor
    kt = O.permute(H.from_array(k.astype(np.float32)), (0, 2, 1))
    _, dkt = O.matmul_backward(H.from_array(g.astype(np.float32)), H.from_array(q.astype(np.float32)), kt, threads=1)
    dk = O.permute_backward(dkt, (0, 2, 1), (2, 5, 4))
    assert dk.shape == (2, 5, 4)
    np.testing.assert_allclose(dk.numpy(), nk, rtol=2e-4, atol=2e-4)


def test_pointwise_backwards_are_derivatives(oracle):
    """bias + GELU (ops/fused.rs:279-392, tanh form), softmax (ops/norm.rs:95-123) and the bias add
    (ops/elementwise.rs:199-211): each backward against central differences of its own forward."""
    O = oracle
    rng = np.random.default_rng(13)
    H = O.HostTensor
    x = rng.standard_normal((3, 5))
    bias = rng.standard_normal((5,))
    g = rng.standard_normal((3, 5))

    def gelu_loss():
        return float(np.sum(g * O.bias_gelu(H.from_array(x.astype(np.float32)),
                                            H.from_array(bias.astype(np.float32))).numpy().astype(np.float64)))
    dx, dbias = O.bias_gelu_backward(H.from_array(g.astype(np.float32)), H.from_array(x.astype(np.float32)),
                                     H.from_array(bias.astype(np.float32)))
    # the forward runs in f32, so the step is large and the tolerance loose
    np.testing.assert_allclose(dx.numpy(), _numeric_grad(gelu_loss, x, eps=1e-2), rtol=5e-3, atol=5e-3)
    np.testing.assert_allclose(dbias.numpy(), _numeric_grad(gelu_loss, bias, eps=1e-2), rtol=5e-3, atol=5e-3)

    s_in = rng.standard_normal((2, 3, 6))
    gs = rng.standard_normal((2, 3, 6))
    for dim in (-1, 1):
        def sm_loss():
            return float(np.sum(gs * O.softmax(s_in.astype(np.float32), dim).astype(np.float64)))
        sm = O.softmax(s_in.astype(np.float32), dim)
        ds = O.softmax_backward(gs.astype(np.float32), sm, dim)
        np.testing.assert_allclose(ds, _numeric_grad(sm_loss, s_in, eps=1e-2), rtol=5e-3, atol=5e-3)
