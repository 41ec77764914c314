"""GPU parity tests: the CUDA library, called through its C ABI, against the CPU oracle on the
same seeded inputs.  Default mode (3xTF32) must satisfy max|d| <= 1e-5 * K * max|a| * max|b|;
the fast TF32 mode is held to a relative Frobenius error of 2e-3."""
import numpy as np
import pytest

from conftest import Guarded, regression_bound_3xtf32, rel_fro, tol_3xtf32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import framework_b200 as F
    F._lib.lib()   # raises if the CUDA library is missing: there is no fallback
    return F


def _dev(F, arr):
    return F.DeviceTensor.from_numpy(arr)


def _check_fwd(F, O, a, b, *, perm_a=None, perm_b=None, bias=None, flags=0, fast=False):
    """a, b: numpy arrays in storage layout; perm_*: stride-only permutation applied on both sides."""
    ha, hb = O.HostTensor.from_array(a), O.HostTensor.from_array(b)
    da, db = _dev(F, a), _dev(F, b)
    if perm_a is not None:
        ha, da = O.permute(ha, perm_a), da.permute(perm_a)
    if perm_b is not None:
        hb, db = O.permute(hb, perm_b), db.permute(perm_b)
    ref = O.matmul(ha, hb)
    if bias is not None:
        ref = O.add(ref, O.HostTensor.from_array(bias))
    gout = Guarded(F, tuple(ref.shape))
    out = F.matmul(da, db, _dev(F, bias) if bias is not None else None, flags=flags, out=gout.tensor)
    F.device_status()
    gout.check("matmul output")
    got = out.numpy()
    assert got.shape == tuple(ref.shape)
    refn = ref.numpy()
    k = ha.shape[-1]
    if fast:
        assert rel_fro(got, refn) <= 2e-3
    else:
        bound = tol_3xtf32(k, a, b) + (1e-6 * np.max(np.abs(bias)) if bias is not None else 0)
        err = float(np.max(np.abs(got - refn))) if got.size else 0.0
        assert err <= bound, f"max err {err:.3e} > bound {bound:.3e} for {a.shape} x {b.shape}"
        if got.size >= 256 and k >= 8:      # the regression bound: what the split really delivers
            assert rel_fro(got, refn) <= regression_bound_3xtf32(k), (rel_fro(got, refn), a.shape, b.shape)
    return got


def _check_bwd(F, O, a, b, g, *, perm_a=None, perm_b=None, flags=0, dbias=False):
    ha, hb, hg = O.HostTensor.from_array(a), O.HostTensor.from_array(b), O.HostTensor.from_array(g)
    da, db, dg = _dev(F, a), _dev(F, b), _dev(F, g)
    if perm_a is not None:
        ha, da = O.permute(ha, perm_a), da.permute(perm_a)
    if perm_b is not None:
        hb, db = O.permute(hb, perm_b), db.permute(perm_b)
    ra, rb = O.matmul_backward(hg, ha, hb)
    g_da, g_db = Guarded(F, tuple(ha.shape)), Guarded(F, tuple(hb.shape))
    g_dbias = Guarded(F, (hb.shape[-1],)) if dbias else None
    res = F.matmul_backward(dg, da, db, flags=flags, want_dbias=dbias, da=g_da.tensor, db=g_db.tensor,
                            dbias=g_dbias.tensor if dbias else None)
    F.device_status()
    g_da.check("grad_a")
    g_db.check("grad_b")
    if dbias:
        g_dbias.check("dbias")
    ga, gb = res[0].numpy(), res[1].numpy()
    m, k, n = ha.shape[-2], ha.shape[-1], hb.shape[-1]
    batch_a = int(np.prod(ha.shape[:-2])) if len(ha.shape) > 2 else 1
    batch_b = int(np.prod(hb.shape[:-2])) if len(hb.shape) > 2 else 1
    batch_g = int(np.prod(hg.shape[:-2])) if len(hg.shape) > 2 else 1
    ka = n * max(1, batch_g // max(batch_a, 1))
    kb = m * max(1, batch_g // max(batch_b, 1))
    ea = float(np.max(np.abs(ga - ra.numpy())))
    eb = float(np.max(np.abs(gb - rb.numpy())))
    assert ea <= tol_3xtf32(ka, g, b), f"dA err {ea:.3e}"
    assert eb <= tol_3xtf32(kb, a, g), f"dB err {eb:.3e}"
    if not (flags & F._lib.PRECISION_TF32):
        if ga.size >= 256 and ka >= 8:
            assert rel_fro(ga, ra.numpy()) <= regression_bound_3xtf32(ka), ("dA", rel_fro(ga, ra.numpy()))
        if gb.size >= 256 and kb >= 8:
            assert rel_fro(gb, rb.numpy()) <= regression_bound_3xtf32(kb), ("dB", rel_fro(gb, rb.numpy()))
    if dbias:
        _, rbias = O.add_backward(hg, hg.shape, (n,))
        ebias = float(np.max(np.abs(res[2].numpy() - rbias.numpy())))
        assert ebias <= 1e-5 * (g.size // n) * float(np.max(np.abs(g)))
    return ga, gb


# ---------------------------------------------------------------------------------------------
def test_reference_known_answers(F, oracle, golden):
    for case in golden["forward"]:
        a = np.array(case["a"]["data"], np.float32).reshape(case["a"]["shape"])
        b = np.array(case["b"]["data"], np.float32).reshape(case["b"]["shape"])
        for flags in (0, F._lib.FORCE_TENSOR_PATH):
            got = F.matmul(_dev(F, a), _dev(F, b), flags=flags).numpy()
            if "data" in case["out"]:
                np.testing.assert_allclose(got.ravel(), case["out"]["data"], atol=case["tol"])
            else:
                assert abs(got.ravel()[0] - case["out"]["first"]) <= case["tol"]
    for case in golden["backward"]:
        a = np.array(case["a"]["data"], np.float32).reshape(case["a"]["shape"])
        b = np.array(case["b"]["data"], np.float32).reshape(case["b"]["shape"])
        g = np.array(case["grad"]["data"], np.float32).reshape(case["grad"]["shape"])
        for flags in (0, F._lib.FORCE_TENSOR_PATH):
            da, db = F.matmul_backward(_dev(F, g), _dev(F, a), _dev(F, b), flags=flags)
            np.testing.assert_allclose(da.numpy().ravel(), case["da"], atol=1e-3)
            np.testing.assert_allclose(db.numpy().ravel(), case["db"], atol=1e-3)


def test_reference_shapes(F, golden):
    rng = np.random.default_rng(0)
    for case in golden["forward_shapes"]:
        a = _dev(F, rng.random(case["a"], dtype=np.float32))
        b = _dev(F, rng.random(case["b"], dtype=np.float32))
        out = F.matmul(a, b)
        if "bias" in case:
            out = F.add(out, _dev(F, rng.random(case["bias"], dtype=np.float32)))
        assert list(out.shape) == case["out"]


def test_config1_square_512(F, oracle):
    """A[512,512].B[512,512] ~N(0,1), seed 0, backward with dC = ones."""
    rng = np.random.default_rng(0)
    a = rng.standard_normal((512, 512), dtype=np.float32)
    b = rng.standard_normal((512, 512), dtype=np.float32)
    _check_fwd(F, oracle, a, b)
    _check_bwd(F, oracle, a, b, np.ones((512, 512), np.float32))


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (2, 3, 7), (17, 33, 9), (31, 64, 65), (128, 128, 32),
                                   (129, 130, 36), (127, 255, 100), (200, 300, 64), (256, 257, 132),
                                   (64, 520, 40), (300, 72, 260)])
def test_odd_shapes_fwd_bwd(F, oracle, m, n, k):
    rng = np.random.default_rng(m * 10007 + n * 101 + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    g = rng.standard_normal((m, n), dtype=np.float32)
    flags = F._lib.FORCE_TENSOR_PATH
    _check_fwd(F, oracle, a, b, flags=flags)
    _check_bwd(F, oracle, a, b, g, flags=flags, dbias=True)


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_all_four_major_combinations(F, oracle, ta, tb):
    """Transposed operands are stride-only views: the kernel reads them through its descriptors."""
    rng = np.random.default_rng(11)
    m, k, n = 192, 160, 320
    a = rng.standard_normal((k, m) if ta else (m, k), dtype=np.float32)
    b = rng.standard_normal((n, k) if tb else (k, n), dtype=np.float32)
    _check_fwd(F, oracle, a, b, perm_a=[1, 0] if ta else None, perm_b=[1, 0] if tb else None,
               flags=F._lib.FORCE_TENSOR_PATH)
    g = rng.standard_normal((m, n), dtype=np.float32)
    _check_bwd(F, oracle, a, b, g, perm_a=[1, 0] if ta else None, perm_b=[1, 0] if tb else None,
               flags=F._lib.FORCE_TENSOR_PATH)


def test_batched_and_broadcast(F, oracle):
    rng = np.random.default_rng(12)
    a = rng.standard_normal((4, 3, 40, 24), dtype=np.float32)
    b = rng.standard_normal((4, 3, 24, 56), dtype=np.float32)
    _check_fwd(F, oracle, a, b)
    _check_bwd(F, oracle, a, b, rng.standard_normal((4, 3, 40, 56), dtype=np.float32))
    w = rng.standard_normal((24, 56), dtype=np.float32)          # shared weight
    _check_fwd(F, oracle, a, w)
    _check_bwd(F, oracle, a, w, rng.standard_normal((4, 3, 40, 56), dtype=np.float32))
    x = rng.standard_normal((40, 24), dtype=np.float32)          # shared left operand
    _check_fwd(F, oracle, x, b)
    _check_bwd(F, oracle, x, b, rng.standard_normal((4, 3, 40, 56), dtype=np.float32))


def test_non_simple_broadcast_matches_reference_indexing(F, oracle):
    rng = np.random.default_rng(13)
    a = rng.standard_normal((2, 1, 20, 12), dtype=np.float32)
    b = rng.standard_normal((1, 3, 12, 28), dtype=np.float32)
    _check_fwd(F, oracle, a, b)
    _check_bwd(F, oracle, a, b, rng.standard_normal((2, 3, 20, 28), dtype=np.float32))


def test_attention_shaped_strided_k(F, oracle):
    """Config 3 at reduced size: S = Q.K^T with K^T a permute(0,1,3,2) view, then S.V, and backward."""
    rng = np.random.default_rng(14)
    bsz, h, s, d = 2, 3, 128, 64
    q = rng.standard_normal((bsz, h, s, d), dtype=np.float32)
    k = rng.standard_normal((bsz, h, s, d), dtype=np.float32)
    v = rng.standard_normal((bsz, h, s, d), dtype=np.float32)
    sc = _check_fwd(F, oracle, q, k, perm_b=[0, 1, 3, 2])
    _check_fwd(F, oracle, sc, v)
    d_o = rng.standard_normal((bsz, h, s, d), dtype=np.float32)
    d_s, _ = _check_bwd(F, oracle, sc, v, d_o)
    _check_bwd(F, oracle, q, k, d_s, perm_b=[0, 1, 3, 2])


def test_permute_backward_returns_the_original_layout(F, oracle):
    """dK of the attention-shaped case: the gradient of K^T = permute(K, [0,1,3,2]) put back in K's layout
    (ops/layout.rs:162-212), bit-exact (it only moves data)."""
    rng = np.random.default_rng(24)
    for shape, dims in (((2, 3, 40, 24), [0, 1, 3, 2]), ((5, 6, 7), [2, 0, 1]), ((9, 4), [1, 0])):
        g = rng.standard_normal([shape[d] for d in dims], dtype=np.float32)
        ref = oracle.permute_backward(oracle.HostTensor.from_array(g), dims, shape).numpy()
        got = F.permute_backward(_dev(F, g), dims, shape)
        assert got.is_contiguous() and got.shape == tuple(shape)
        assert np.array_equal(got.numpy(), ref)
    dev = _dev(F, rng.standard_normal((6, 8, 10), dtype=np.float32))
    view = F.permute(dev, [1, 2, 0])
    assert view.ptr == dev.ptr and view.strides == (10, 1, 80) and not view.is_contiguous()
    assert np.array_equal(view.contiguous().numpy(), np.transpose(dev.numpy(), (1, 2, 0)))


def test_head_split_view_with_two_batch_strides(F, oracle):
    """[B,S,H,D] -> permute(0,2,1,3): batch dims that do not collapse into one stride."""
    rng = np.random.default_rng(15)
    x = rng.standard_normal((2, 48, 3, 32), dtype=np.float32)
    w = rng.standard_normal((2, 3, 32, 40), dtype=np.float32)
    _check_fwd(F, oracle, x, w, perm_a=[0, 2, 1, 3])
    _check_bwd(F, oracle, x, w, rng.standard_normal((2, 3, 48, 40), dtype=np.float32), perm_a=[0, 2, 1, 3])


def test_linear_layer_fused_and_drop_in(F, oracle):
    """Config 2 at reduced size: y = x.W + b, backward gives dx, dW, db."""
    rng = np.random.default_rng(16)
    x = rng.random((384, 256), dtype=np.float32)
    w = (0.02 * rng.standard_normal((256, 512))).astype(np.float32)
    dy = rng.standard_normal((384, 512), dtype=np.float32)
    for bias in (np.zeros(512, np.float32), (0.02 * rng.standard_normal(512)).astype(np.float32)):
        fused = _check_fwd(F, oracle, x, w, bias=bias)
        lin = F.Linear(_dev(F, w), _dev(F, bias))
        two_step = lin.forward(_dev(F, x)).numpy()
        assert float(np.max(np.abs(two_step - fused))) <= 1e-6
    _check_bwd(F, oracle, x, w, dy, dbias=True)
    ga, gb = F.add_backward(_dev(F, dy), dy.shape, (512,))
    ra, rb = oracle.add_backward(oracle.HostTensor.from_array(dy), dy.shape, (512,))
    assert np.array_equal(ga.numpy(), ra.numpy())
    assert float(np.max(np.abs(gb.numpy() - rb.numpy()))) <= 1e-5 * 384 * float(np.max(np.abs(dy)))


def test_broadcast_weight_gradient_is_reduced_in_the_gemm(F, oracle):
    """Config 4 at reduced size: dW sums over the batch broadcast."""
    rng = np.random.default_rng(17)
    a = rng.standard_normal((6, 100, 96), dtype=np.float32)
    w = (0.02 * rng.standard_normal((96, 200))).astype(np.float32)
    _check_fwd(F, oracle, a, w)
    _check_bwd(F, oracle, a, w, rng.standard_normal((6, 100, 200), dtype=np.float32))


@pytest.mark.parametrize("m", [1, 4, 16])
def test_skinny_rows(F, oracle, m):
    """Config 5b at reduced size, on the skinny path and forced onto the tensor path."""
    rng = np.random.default_rng(18 + m)
    x = rng.standard_normal((m, 512), dtype=np.float32)
    w = rng.standard_normal((512, 768), dtype=np.float32)
    dy = rng.standard_normal((m, 768), dtype=np.float32)
    for flags in (0, F._lib.FORCE_TENSOR_PATH):
        _check_fwd(F, oracle, x, w, flags=flags)
        _check_bwd(F, oracle, x, w, dy, flags=flags)
    bias = rng.standard_normal(768, dtype=np.float32)
    _check_fwd(F, oracle, x, w, bias=bias)


@pytest.mark.parametrize("m,k,n", [(1, 1024, 1024), (2, 333, 260), (3, 64, 128), (5, 1000, 516), (8, 2048, 512),
                                   (13, 777, 1284), (16, 1, 4), (16, 640, 256), (7, 37, 8), (6, 515, 514),
                                   (8, 90, 1023), (2, 4100, 36)])
def test_streaming_forward_kernels_for_every_row_count(F, oracle, m, k, n):
    """The forced streaming forward (both of its kernels: the cp.async-ring one needs N % 4 == 0) against the
    oracle: contraction lengths that leave ragged k slices, strips narrower than a block, bias, accumulation,
    and a second call that must find the finish tickets clean."""
    rng = np.random.default_rng(300 + m + k + n)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    skinny = F._lib.FORCE_SKINNY_PATH
    first = _check_fwd(F, oracle, x, w, flags=skinny)
    again = _check_fwd(F, oracle, x, w, flags=skinny)
    assert np.array_equal(first, again)            # fixed summation order
    with_bias = _check_fwd(F, oracle, x, w, bias=bias, flags=skinny)
    # c += a.b + bias on top of a known c
    c0 = rng.standard_normal((m, n), dtype=np.float32)
    out = _dev(F, c0)
    F.matmul(_dev(F, x), _dev(F, w), _dev(F, bias), flags=skinny | F._lib.ACCUMULATE_C, out=out)
    F.device_status()
    assert np.max(np.abs(out.numpy() - (c0 + with_bias))) <= 1e-5 * max(1.0, float(np.max(np.abs(with_bias))))


@pytest.mark.parametrize("m,k,n", [(1, 1000, 1024), (2, 333, 260), (3, 67, 128), (4, 1030, 516), (5, 18, 1284),
                                   (7, 515, 512), (8, 2048, 644), (8, 3, 4), (6, 129, 4100)])
def test_streaming_backward_kernels_for_every_row_count(F, oracle, m, k, n):
    """The forced streaming dx and dW kernels against the oracle: row counts on both sides of the switch between
    the two dx kernels, K that is not a multiple of a block's rows, N that is not a multiple of a warp's 128-column
    step; then the same call accumulating onto known gradients."""
    rng = np.random.default_rng(500 + m + k + n)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((k, n), dtype=np.float32)
    dy = rng.standard_normal((m, n), dtype=np.float32)
    skinny = F._lib.FORCE_SKINNY_PATH
    ga, gb = _check_bwd(F, oracle, x, w, dy, flags=skinny)
    a0 = rng.standard_normal((m, k), dtype=np.float32)
    b0 = rng.standard_normal((k, n), dtype=np.float32)
    da, db = _dev(F, a0), _dev(F, b0)
    F.matmul_backward(_dev(F, dy), _dev(F, x), _dev(F, w), da=da, db=db,
                      flags=skinny | F._lib.ACCUMULATE_DA | F._lib.ACCUMULATE_DB)
    F.device_status()
    assert np.max(np.abs(da.numpy() - (a0 + ga))) <= 1e-5 * max(1.0, float(np.max(np.abs(ga))))
    assert np.max(np.abs(db.numpy() - (b0 + gb))) <= 1e-5 * max(1.0, float(np.max(np.abs(gb))))


def test_forced_split_k_and_pack_paths(F, oracle):
    rng = np.random.default_rng(19)
    a = rng.standard_normal((150, 700), dtype=np.float32)
    b = rng.standard_normal((700, 90), dtype=np.float32)
    for flags in (F._lib.force_split_k(3), F._lib.force_split_k(7), F._lib.FORCE_PACK,
                  F._lib.FORCE_PACK | F._lib.force_split_k(2)):
        _check_fwd(F, oracle, a, b, flags=flags | F._lib.FORCE_TENSOR_PATH)
    _check_fwd(F, oracle, a, b, bias=rng.standard_normal(90, dtype=np.float32),
               flags=F._lib.force_split_k(4) | F._lib.FORCE_TENSOR_PATH)


def test_accumulate_flags(F, oracle):
    rng = np.random.default_rng(20)
    a = rng.standard_normal((70, 50), dtype=np.float32)
    b = rng.standard_normal((50, 60), dtype=np.float32)
    g = rng.standard_normal((70, 60), dtype=np.float32)
    base_c = rng.standard_normal((70, 60), dtype=np.float32)
    out = _dev(F, base_c)
    F.matmul(_dev(F, a), _dev(F, b), flags=F._lib.ACCUMULATE_C | F._lib.FORCE_TENSOR_PATH, out=out)
    ref = base_c + oracle.matmul(oracle.HostTensor.from_array(a), oracle.HostTensor.from_array(b)).numpy()
    assert float(np.max(np.abs(out.numpy() - ref))) <= tol_3xtf32(50, a, b)
    base_a, base_b = rng.standard_normal(a.shape, dtype=np.float32), rng.standard_normal(b.shape, dtype=np.float32)
    da, db = _dev(F, base_a), _dev(F, base_b)
    F.matmul_backward(_dev(F, g), _dev(F, a), _dev(F, b), da=da, db=db,
                      flags=F._lib.ACCUMULATE_DA | F._lib.ACCUMULATE_DB | F._lib.FORCE_TENSOR_PATH)
    ra, rb = oracle.matmul_backward(oracle.HostTensor.from_array(g), oracle.HostTensor.from_array(a),
                                    oracle.HostTensor.from_array(b))
    assert float(np.max(np.abs(da.numpy() - (base_a + ra.numpy())))) <= tol_3xtf32(60, g, b)
    assert float(np.max(np.abs(db.numpy() - (base_b + rb.numpy())))) <= tol_3xtf32(70, a, g)


def test_fast_tf32_mode(F, oracle):
    rng = np.random.default_rng(21)
    a = rng.standard_normal((256, 384), dtype=np.float32)
    b = rng.standard_normal((384, 320), dtype=np.float32)
    _check_fwd(F, oracle, a, b, flags=F._lib.PRECISION_TF32 | F._lib.FORCE_TENSOR_PATH, fast=True)


def test_tensor_core_ignores_low_mantissa_bits(F):
    """The 3xTF32 split uses the raw f32 tile as its "hi" part, which is only right if the tensor core
    truncates (ignores the low 13 mantissa bits of) a TF32 operand.  Pin that: single-pass TF32 on raw
    inputs must be bit-identical to single-pass TF32 on inputs whose low 13 bits were cleared."""
    rng = np.random.default_rng(23)
    a = rng.standard_normal((256, 192), dtype=np.float32)
    b = rng.standard_normal((192, 320), dtype=np.float32)
    mask = np.uint32(0xFFFFE000)
    am = (a.view(np.uint32) & mask).view(np.float32)
    bm = (b.view(np.uint32) & mask).view(np.float32)
    flags = F._lib.PRECISION_TF32 | F._lib.FORCE_TENSOR_PATH
    raw = F.matmul(_dev(F, a), _dev(F, b), flags=flags).numpy()
    cut = F.matmul(_dev(F, am), _dev(F, bm), flags=flags).numpy()
    F.device_status()
    assert np.array_equal(raw, cut)
    for perm_a, perm_b in (([1, 0], None), (None, [1, 0])):     # MN-major A, K-major B
        at, bt = np.ascontiguousarray(a.T), np.ascontiguousarray(b.T)
        atm, btm = np.ascontiguousarray(am.T), np.ascontiguousarray(bm.T)
        x = _dev(F, at).permute(perm_a) if perm_a else _dev(F, a)
        y = _dev(F, bt).permute(perm_b) if perm_b else _dev(F, b)
        xm = _dev(F, atm).permute(perm_a) if perm_a else _dev(F, am)
        ym = _dev(F, btm).permute(perm_b) if perm_b else _dev(F, bm)
        assert np.array_equal(F.matmul(x, y, flags=flags).numpy(), F.matmul(xm, ym, flags=flags).numpy())


def test_outputs_are_fully_overwritten(F, oracle):
    """store.zeros may hand back a dirty buffer (allocator.rs:61-66): stale contents must not leak."""
    import torch
    rng = np.random.default_rng(22)
    a = rng.standard_normal((100, 36), dtype=np.float32)
    b = rng.standard_normal((36, 44), dtype=np.float32)
    out = F.DeviceTensor(torch.full((100 * 44,), float("nan"), device="cuda"), (100, 44))
    F.matmul(_dev(F, a), _dev(F, b), out=out, flags=F._lib.FORCE_TENSOR_PATH)
    assert np.isfinite(out.numpy()).all()


def test_empty_and_degenerate(F, oracle):
    a0 = F.DeviceTensor.empty((0, 8))
    b = _dev(F, np.ones((8, 4), np.float32))
    assert F.matmul(a0, b).shape == (0, 4)
    az = F.DeviceTensor.empty((5, 0))
    bz = F.DeviceTensor.empty((0, 4))
    out = F.matmul(az, bz)
    assert out.shape == (5, 4) and not out.numpy().any()


def test_linearity_at_full_size_config2(F):
    """Size-independent property at the bench workload's full size: (a1 + a2).W == a1.W + a2.W."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(0)
    x1 = torch.rand((4096, 1024), device="cuda", generator=g)
    x2 = torch.rand((4096, 1024), device="cuda", generator=g)
    w = 0.02 * torch.randn((1024, 4096), device="cuda", generator=g)
    t = F.DeviceTensor.from_torch
    y12 = F.matmul(t(x1 + x2), t(w)).torch_view()
    y1 = F.matmul(t(x1), t(w)).torch_view()
    y2 = F.matmul(t(x2), t(w)).torch_view()
    F.device_status()
    bound = 1e-5 * 1024 * 2.0 * float(w.abs().max())
    assert float((y12 - y1 - y2).abs().max()) <= 3 * bound
    ref = (x1.double() @ w.double())
    assert float((y1.double() - ref).abs().max()) <= 1e-5 * 1024 * 1.0 * float(w.abs().max())


def test_small_backward_side_stream_inside_a_cuda_graph(F, oracle):
    """A small backward issues grad_b on the library's side stream (fork/join through events).  Captured into a
    CUDA graph and replayed twice with new inputs, both gradients must still match the oracle."""
    import torch
    rng = np.random.default_rng(21)
    a = rng.standard_normal((96, 80), dtype=np.float32)
    b = rng.standard_normal((80, 72), dtype=np.float32)
    g = rng.standard_normal((96, 72), dtype=np.float32)
    ad, bd, gd = (F.DeviceTensor.from_numpy(x) for x in (a, b, g))
    da, db = F.DeviceTensor.empty(a.shape), F.DeviceTensor.empty(b.shape)
    F.matmul_backward(gd, ad, bd, da=da, db=db)            # eager once: scratch is sized before capture
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            F.matmul_backward(gd, ad, bd, da=da, db=db)
    for seed in (1, 2):
        g2 = np.random.default_rng(seed).standard_normal(g.shape, dtype=np.float32)
        gd.storage.copy_(torch.from_numpy(g2.ravel()))
        da.storage.zero_(); db.storage.zero_()
        graph.replay()
        torch.cuda.synchronize()
        H = oracle.HostTensor
        ra, rb = oracle.matmul_backward(H.from_array(g2), H.from_array(a), H.from_array(b))
        assert np.max(np.abs(da.numpy() - ra.numpy())) <= tol_3xtf32(72, g2, b)
        assert np.max(np.abs(db.numpy() - rb.numpy())) <= tol_3xtf32(96, a, g2)
    F.device_status()


@pytest.mark.parametrize("m,k,n", [(256, 512, 16), (300, 200, 24), (128, 2048, 40), (384, 96, 8)])
@pytest.mark.parametrize("b_transposed", [False, True])
def test_narrow_outputs_multiply_only_live_columns(F, oracle, m, k, n, b_transposed):
    """Tiles wider than the output: the MMAs are issued N-wide (in units of 16, or whole 32-float chunks when B is
    read along N), and for a B that is contiguous along the contraction only its live rows are loaded and split.
    The accumulator columns beyond are never written, so nothing of them may reach the output: plain forward,
    with bias, accumulated onto a non-zero C, with a forced split of the contraction, single pass, and both
    gradients -- all inside guard zones."""
    rng = np.random.default_rng(1000 * n + m)
    a = rng.standard_normal((m, k), dtype=np.float32)
    bias = rng.standard_normal((n,), dtype=np.float32)
    T = F._lib.FORCE_TENSOR_PATH
    if b_transposed:                              # storage [n, k]: rows contiguous along the contraction
        b = rng.standard_normal((n, k), dtype=np.float32)
        perm = (1, 0)
    else:
        b = rng.standard_normal((k, n), dtype=np.float32)
        perm = None
    for flags, kw in ((T, {}), (T, {"bias": bias}), (T | F._lib.force_split_k(3), {}),
                      (T | F._lib.PRECISION_TF32, {"fast": True})):
        _check_fwd(F, oracle, a, b, perm_b=perm, flags=flags, **kw)
    # C += a.b on a C that holds data
    H = oracle.HostTensor
    hb = H.from_array(b) if perm is None else oracle.permute(H.from_array(b), perm)
    db = _dev(F, b) if perm is None else _dev(F, b).permute(perm)
    c0 = rng.standard_normal((m, n), dtype=np.float32)
    gout = Guarded(F, (m, n), init=c0)
    F.matmul(_dev(F, a), db, flags=T | F._lib.ACCUMULATE_C, out=gout.tensor)
    F.device_status()
    gout.check("accumulated output", fully_written=False)
    ref = oracle.matmul(H.from_array(a), hb).numpy() + c0
    assert float(np.max(np.abs(gout.tensor.numpy() - ref))) <= tol_3xtf32(k, a, b) + 1e-6
    g = rng.standard_normal((m, n), dtype=np.float32)
    _check_bwd(F, oracle, a, b, g, perm_b=perm, flags=T)


def test_plan_description_matches_what_is_launched(F):
    """`plan_describe` (host arithmetic, checked without a device in the CPU tests) names the launches a call
    makes: for tensor-path products the launch counter must move by one per described product, plus one for the
    finish kernel of a split contraction."""
    import re
    import torch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rng = np.random.default_rng(44)
    for a_shape, b_shape in (((512, 512), (512, 512)), ((1024, 768), (768, 1536)), ((6, 256, 64), (6, 64, 256))):
        a = F.DeviceTensor.from_numpy(rng.standard_normal(a_shape, dtype=np.float32))
        b = F.DeviceTensor.from_numpy(rng.standard_normal(b_shape, dtype=np.float32))
        for backward in (0, 1):
            lines = [l for l in F.plan_describe(a_shape, b_shape, backward=backward, sm_count=sms) if "tensor" in l]
            assert len(lines) == (2 if backward else 1), lines
            expect = sum(1 + (int(re.search(r"splits=(\d+)", l).group(1)) > 1) for l in lines)
            before = F.launch_count()
            if backward:
                g = F.DeviceTensor.from_numpy(rng.standard_normal(a_shape[:-1] + b_shape[-1:], dtype=np.float32))
                F.matmul_backward(g, a, b)
            else:
                F.matmul(a, b)
            assert F.launch_count() - before == expect, (a_shape, b_shape, backward, lines)
    F.device_status()


def test_scratch_growth_is_refused_while_a_stream_captures(F, oracle):
    """Growing the library-owned scratch frees the old buffer, which a capturing stream must not do and which
    would leave recorded nodes with a dangling address.  A call that would need it during a capture fails with
    MNI_B200_ERR_WORKSPACE before anything is recorded, the capture itself stays valid, and the same call run
    eagerly afterwards grows the scratch and is correct."""
    import torch
    lib = F._lib.lib()
    rng = np.random.default_rng(33)
    small_a = rng.standard_normal((128, 256), dtype=np.float32)
    small_b = rng.standard_normal((256, 128), dtype=np.float32)
    a = rng.standard_normal((1024, 2048), dtype=np.float32)
    b = rng.standard_normal((2048, 1024), dtype=np.float32)
    sa, sb, ad, bd = (F.DeviceTensor.from_numpy(x) for x in (small_a, small_b, a, b))
    split = F._lib.FORCE_TENSOR_PATH | F._lib.force_split_k(4)
    torch.cuda.synchronize()
    F._lib.check(lib.mni_b200_release())                 # start from no scratch at all
    small = F.matmul(sa, sb, flags=split)                # 4 x 64 KiB of partial sums: a small buffer now exists
    out = F.DeviceTensor.empty((1024, 1024))
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            F.matmul(sa, sb, out=small, flags=split)     # fits: recorded
            with pytest.raises(F._lib.MniError) as ei:   # 4 x 4 MiB of partial sums: would have to grow
                F.matmul(ad, bd, out=out, flags=split)
    assert ei.value.status == 7, ei.value                # MNI_B200_ERR_WORKSPACE
    assert "capturing" in ei.value.message
    small.storage.zero_()
    graph.replay()                                       # the capture survived the refused call
    torch.cuda.synchronize()
    H = oracle.HostTensor
    ref_small = oracle.matmul(H.from_array(small_a), H.from_array(small_b)).numpy()
    assert np.max(np.abs(small.numpy() - ref_small)) <= tol_3xtf32(256, small_a, small_b)
    F.matmul(ad, bd, out=out, flags=split)               # eager: grows and runs
    ref = oracle.matmul(H.from_array(a), H.from_array(b)).numpy()
    assert np.max(np.abs(out.numpy() - ref)) <= tol_3xtf32(2048, a, b)
    F.device_status()


@pytest.mark.parametrize("shape_a,shape_b,flags,bias", [
    ((1536, 512), (512, 2048), 0, False),            # 48 pair-tiles on 74 pairs: every tile is cut 2-3 ways
    ((2560, 1024), (1024, 2304), 0, True),           # one whole round, then a 16-tile tail dealt out by k-blocks
    ((24, 512, 512), (24, 512, 64), 0, False),       # 64-wide tiles (A from tensor memory), 96 tiles on 148 CTAs
    ((1536, 512), (512, 2048), 1, False),            # single-pass TF32 mode
])
def test_balanced_tail_matches_oracle(F, oracle, monkeypatch, shape_a, shape_b, flags, bias):
    """Shapes whose last wave of tiles is ragged, with the balanced tail switched on (it is opt-in): the tail's
    k-blocks are dealt out evenly and a tile shared by several CTAs is summed in the epilogue of the last one
    to arrive.  Forward (with bias) and both gradients against the CPU backend."""
    monkeypatch.setenv("MNI_B200_STREAMK", "1")
    rng = np.random.default_rng(sum(shape_a) + sum(shape_b))
    a = rng.standard_normal(shape_a, dtype=np.float32)
    b = rng.standard_normal(shape_b, dtype=np.float32)
    bv = rng.standard_normal(shape_b[-1], dtype=np.float32) if bias else None
    H = oracle.HostTensor
    ref = oracle.matmul(H.from_array(a), H.from_array(b)).numpy()
    if bias:
        ref = ref + bv
    out = F.matmul(F.DeviceTensor.from_numpy(a), F.DeviceTensor.from_numpy(b),
                   F.DeviceTensor.from_numpy(bv) if bias else None, flags=flags)
    F.device_status()
    k = shape_a[-1]
    if flags & 1:
        assert rel_fro(out.numpy(), ref) <= 2e-3
    else:
        assert float(np.max(np.abs(out.numpy() - ref))) <= tol_3xtf32(k, a, b) + 1e-6
    g = rng.standard_normal(ref.shape, dtype=np.float32)
    da, db = F.matmul_backward(F.DeviceTensor.from_numpy(g), F.DeviceTensor.from_numpy(a), F.DeviceTensor.from_numpy(b),
                               flags=flags)
    F.device_status()
    ra, rb = oracle.matmul_backward(H.from_array(g), H.from_array(a), H.from_array(b))
    if flags & 1:
        assert rel_fro(da.numpy(), ra.numpy()) <= 2e-3 and rel_fro(db.numpy(), rb.numpy()) <= 2e-3
    else:
        assert float(np.max(np.abs(da.numpy() - ra.numpy()))) <= tol_3xtf32(shape_b[-1], g, b)
        kb = shape_a[-2] * (int(np.prod(shape_a[:-2])) if len(shape_b) == 2 else 1)
        assert float(np.max(np.abs(db.numpy() - rb.numpy()))) <= tol_3xtf32(kb, a, g)


def test_balanced_tail_is_reproducible_and_leaves_flags_clear(F, monkeypatch):
    """Two runs of a cut-tile product are bit-identical (fixed summation order, whoever arrives last) and so is a
    third after other launches: tickets and ready flags are cleared by the reducing CTA.  The result also agrees
    with the whole-tile schedule to rounding."""
    monkeypatch.setenv("MNI_B200_STREAMK", "1")
    rng = np.random.default_rng(77)
    a = F.DeviceTensor.from_numpy(rng.standard_normal((1536, 512), dtype=np.float32))
    b = F.DeviceTensor.from_numpy(rng.standard_normal((512, 2048), dtype=np.float32))
    first = F.matmul(a, b).numpy()
    second = F.matmul(a, b).numpy()
    F.matmul(b.permute((1, 0)), a.permute((1, 0)))          # another cut-tile launch in between
    third = F.matmul(a, b).numpy()
    F.device_status()
    assert np.array_equal(first, second) and np.array_equal(first, third)
    monkeypatch.setenv("MNI_B200_STREAMK", "0")
    whole = F.matmul(a, b).numpy()
    assert rel_fro(first, whole) < 1e-5          # two summation orders of 3xTF32 products


@pytest.mark.parametrize("m,k,n,batch", [(40, 300, 512, ()), (64, 512, 512, (3,)), (16, 1024, 2048, ()), (33, 96, 260, (2, 2))])
def test_few_rows_many_columns_is_computed_transposed(F, oracle, m, k, n, batch):
    """M <= 64 with N >= 256: the kernel computes C^T with the operands exchanged and stores transposed patches
    (bias then runs along the kernel's rows).  Forward with bias, accumulate, a forced K split and both
    gradients against the CPU backend."""
    rng = np.random.default_rng(m * 1000 + n)
    a = rng.standard_normal(batch + (m, k), dtype=np.float32)
    b = rng.standard_normal(batch + (k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    H = oracle.HostTensor
    ref = oracle.matmul(H.from_array(a), H.from_array(b)).numpy()
    ad, bd, biasd = (F.DeviceTensor.from_numpy(x) for x in (a, b, bias))
    tol = tol_3xtf32(k, a, b) + 1e-5
    for flags in (F._lib.FORCE_TENSOR_PATH, F._lib.FORCE_TENSOR_PATH | (3 << 16)):
        out = F.matmul(ad, bd, biasd, flags=flags)
        F.device_status()
        assert float(np.max(np.abs(out.numpy() - (ref + bias)))) <= tol, hex(flags)
    base = rng.standard_normal(ref.shape, dtype=np.float32)
    out = F.DeviceTensor.from_numpy(base)
    F.matmul(ad, bd, out=out, flags=F._lib.FORCE_TENSOR_PATH | F._lib.ACCUMULATE_C)
    assert float(np.max(np.abs(out.numpy() - (base + ref)))) <= tol
    g = rng.standard_normal(ref.shape, dtype=np.float32)
    da, db = F.matmul_backward(F.DeviceTensor.from_numpy(g), ad, bd, flags=F._lib.FORCE_TENSOR_PATH)
    F.device_status()
    ra, rb = oracle.matmul_backward(H.from_array(g), H.from_array(a), H.from_array(b))
    assert float(np.max(np.abs(da.numpy() - ra.numpy()))) <= tol_3xtf32(n, g, b)
    assert float(np.max(np.abs(db.numpy() - rb.numpy()))) <= tol_3xtf32(m, a, g)


@pytest.mark.parametrize("shape_a,shape_b", [((512, 512), (512, 512)), ((1536, 512), (512, 2048)), ((6, 100, 96), (96, 200)),
                                             ((150, 700), (700, 90)), ((4, 3, 40, 24), (4, 3, 24, 56))])
def test_independent_pair_launch_of_the_two_gradients(F, oracle, monkeypatch, shape_a, shape_b):
    """MNI_B200_BWD_PAIR=1: grad_a and grad_b as an independent pair on one stream (the second product skips its
    dependency wait, runs beside the first and waits for it before it ends).  Called three times in a row with new
    output gradients, so that a second product that started before its inputs were ready, or a following call that
    did not wait for the first product, would show."""
    monkeypatch.setenv("MNI_B200_BWD_PAIR", "1")
    rng = np.random.default_rng(sum(shape_a))
    a = rng.standard_normal(shape_a, dtype=np.float32)
    b = rng.standard_normal(shape_b, dtype=np.float32)
    for _ in range(3):
        g = rng.standard_normal(shape_a[:-1] + (shape_b[-1],), dtype=np.float32)
        _check_bwd(F, oracle, a, b, g, flags=F._lib.FORCE_TENSOR_PATH)
    _check_bwd(F, oracle, a, b, g, flags=F._lib.FORCE_TENSOR_PATH | F._lib.force_split_k(2))
    _check_bwd(F, oracle, a, b, g, flags=F._lib.FORCE_TENSOR_PATH | F._lib.FORCE_PACK)


@pytest.mark.parametrize("m,k,n", [(1, 1000, 1024), (2, 333, 260), (3, 67, 128), (4, 4096, 4096), (5, 18, 1284),
                                   (7, 515, 512), (8, 2048, 644), (8, 3, 4), (6, 129, 4100)])
def test_sliced_streaming_dx_kernel(F, oracle, monkeypatch, m, k, n):
    """The opt-in dx kernel (a block owns 16 weight rows, each warp a slice of N whose dy values stay in
    registers): every row count, ragged K and N, accumulation; bit-identical on a second call."""
    monkeypatch.setenv("MNI_B200_SKINNY_DX_SLICED", "1")
    rng = np.random.default_rng(700 + m + k + n)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((k, n), dtype=np.float32)
    dy = rng.standard_normal((m, n), dtype=np.float32)
    skinny = F._lib.FORCE_SKINNY_PATH
    for variant in ("0", "1", "2"):
        monkeypatch.setenv("MNI_B200_DXS_VARIANT", variant)
        ga, _ = _check_bwd(F, oracle, x, w, dy, flags=skinny)
        again, _ = _check_bwd(F, oracle, x, w, dy, flags=skinny)
        assert np.array_equal(ga, again)
    a0 = rng.standard_normal((m, k), dtype=np.float32)
    da = _dev(F, a0)
    F.matmul_backward(_dev(F, dy), _dev(F, x), _dev(F, w), da=da, need_db=False, flags=skinny | F._lib.ACCUMULATE_DA)
    F.device_status()
    assert np.max(np.abs(da.numpy() - (a0 + ga))) <= 1e-5 * max(1.0, float(np.max(np.abs(ga))))


def test_sm_reservation_leaves_results_unchanged(F, oracle):
    """mni_b200_sm_reserve keeps SMs out of the persistent grids (room for a collective that runs beside a
    product): plans change (fewer slots, other splits / tails), results must not, and 0 restores the full grid."""
    rng = np.random.default_rng(91)
    shapes = [((1536, 512), (512, 2048)), ((6, 100, 96), (96, 200)), ((512, 512), (512, 512)), ((300, 72), (72, 260))]
    try:
        for reserve in (16, 64, 0):
            F.sm_reserve(reserve)
            for sa, sb in shapes:
                a = rng.standard_normal(sa, dtype=np.float32)
                b = rng.standard_normal(sb, dtype=np.float32)
                g = rng.standard_normal(sa[:-1] + (sb[-1],), dtype=np.float32)
                _check_fwd(F, oracle, a, b, flags=F._lib.FORCE_TENSOR_PATH)
                _check_bwd(F, oracle, a, b, g, flags=F._lib.FORCE_TENSOR_PATH)
    finally:
        F.sm_reserve(0)
    with pytest.raises(F._lib.MniError):
        F.sm_reserve(-1)


def test_weight_gradient_in_row_panels_through_narrow_views(F, oracle):
    """What the row-sharded square problem does for its pipelined reduce: rows [lo, hi) of dB = A[:, lo:hi]^T . dC,
    with the column panel of A and the row panel of B passed as views of the same storage (pointer offset + same
    strides) and each panel's result landing in its rows of ONE flat buffer."""
    import torch
    from framework_b200.sharding import panel_bounds
    rng = np.random.default_rng(92)
    m, k, n = 384, 640, 320
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    g = rng.standard_normal((m, n), dtype=np.float32)
    H = oracle.HostTensor
    _, ref_db = oracle.matmul_backward(H.from_array(g), H.from_array(a), H.from_array(b))
    ad, bd, gd = _dev(F, a), _dev(F, b), _dev(F, g)
    flat = torch.full((k * n,), float("nan"), device="cuda")
    for lo, hi in panel_bounds(k, 3, multiple=128):
        a_cols, b_rows = ad.narrow(1, lo, hi - lo), bd.narrow(0, lo, hi - lo)
        assert a_cols.ptr == ad.ptr + 4 * lo and a_cols.strides == ad.strides and not a_cols.is_contiguous()
        assert b_rows.is_contiguous()
        F.matmul_backward(gd, a_cols, b_rows, need_da=False, db=F.DeviceTensor(flat[lo * n:hi * n], (hi - lo, n)))
    F.device_status()
    got = flat.cpu().numpy().reshape(k, n)
    assert float(np.max(np.abs(got - ref_db.numpy()))) <= tol_3xtf32(m, a, g)
    assert rel_fro(got, ref_db.numpy()) <= regression_bound_3xtf32(m)
    with pytest.raises(ValueError):
        ad.narrow(1, 600, 100)


def test_balanced_tail_with_a_long_contraction(F, oracle, monkeypatch):
    """Tail ranges longer than a tile (K = 2048, 90 pair-tiles on 74 pairs): the whole tiles inside a range are summed
    in pieces like every other unit, the cut ones in one accumulator each.  Acceptance bound, and a relative error
    bound that allows for a cut tile's longer chain (the accumulate truncates: ~7e-9 per contraction element)."""
    monkeypatch.setenv("MNI_B200_STREAMK", "1")
    rng = np.random.default_rng(93)
    a = rng.standard_normal((2560, 2048), dtype=np.float32)
    b = rng.standard_normal((2048, 2304), dtype=np.float32)
    H = oracle.HostTensor
    ref = oracle.matmul(H.from_array(a), H.from_array(b)).numpy()
    first = F.matmul(_dev(F, a), _dev(F, b)).numpy()
    again = F.matmul(_dev(F, a), _dev(F, b)).numpy()
    F.device_status()
    assert np.array_equal(first, again)
    assert float(np.max(np.abs(first - ref))) <= tol_3xtf32(2048, a, b)
    assert rel_fro(first, ref) <= 5e-6 + 1e-8 * 2048


def test_shard_of_the_broadcast_weight_problem_takes_the_default_tail(F, oracle):
    """One rank's share of an 8-rank run of the broadcast-weight configuration ([8,1024,768].[768,3072]): its input
    gradient has 96 pair-tiles for 74 pairs, which the default policy runs with the balanced tail.  First and last
    128 rows of dA against the CPU backend."""
    rng = np.random.default_rng(94)
    a = rng.standard_normal((8, 1024, 768), dtype=np.float32)
    w = (0.02 * rng.standard_normal((768, 3072))).astype(np.float32)
    g = rng.standard_normal((8, 1024, 3072), dtype=np.float32)
    da, _ = F.matmul_backward(_dev(F, g), _dev(F, a), _dev(F, w))
    F.device_status()
    da = da.numpy()
    H = oracle.HostTensor
    wt = oracle.permute(H.from_array(w), [1, 0])
    for bt, rows in ((0, slice(0, 128)), (7, slice(896, 1024))):
        ref = oracle.matmul(H.from_array(g[bt, rows]), wt).numpy()
        assert float(np.max(np.abs(da[bt, rows] - ref))) <= tol_3xtf32(3072, g, w)
        assert rel_fro(da[bt, rows], ref) <= 5e-6 + 1e-8 * 3072
