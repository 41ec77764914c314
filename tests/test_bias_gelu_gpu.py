"""GPU parity of the bias + GELU widening: the stand-alone kernels and the GEMM epilogue that fuses
matmul -> bias_gelu, against the CPU oracle (ops/fused.rs:251-277, :317-352 restated in C)."""
import numpy as np
import pytest

from conftest import tol_3xtf32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import framework_b200 as F
    F._lib.lib()
    return F


def _dev(F, arr):
    return F.DeviceTensor.from_numpy(arr)


@pytest.mark.parametrize("shape", [(64, 128), (33, 30), (4, 5, 96), (1, 7)])
def test_bias_gelu_forward_and_backward(F, oracle, shape):
    rng = np.random.default_rng(sum(shape))
    x = (2.0 * rng.standard_normal(shape)).astype(np.float32)
    bias = rng.standard_normal(shape[-1], dtype=np.float32)
    g = rng.standard_normal(shape, dtype=np.float32)
    H = oracle.HostTensor.from_array
    ref = oracle.bias_gelu(H(x), H(bias)).numpy()
    got = F.bias_gelu(_dev(F, x), _dev(F, bias)).numpy()
    # tanhf of the device and of the host libm differ by a few ulp
    assert float(np.max(np.abs(got - ref))) <= 2e-6 * (1.0 + float(np.abs(x).max() + np.abs(bias).max()))
    rdx, rdb = oracle.bias_gelu_backward(H(g), H(x), H(bias))
    dx, db = F.bias_gelu_backward(_dev(F, g), _dev(F, x), _dev(F, bias))
    F.device_status()
    assert float(np.max(np.abs(dx.numpy() - rdx.numpy()))) <= 4e-6 * float(np.abs(g).max()) * 1.2
    rows = int(np.prod(shape[:-1]))
    assert float(np.max(np.abs(db.numpy() - rdb.numpy()))) <= 1e-5 * rows * float(np.abs(g).max()) * 1.2


@pytest.mark.parametrize("m,k,n,flags_name", [(384, 256, 512, None), (200, 100, 72, None), (130, 64, 30, None),
                                              (4, 256, 512, None), (256, 2048, 256, "split")])
def test_matmul_with_bias_gelu_epilogue(F, oracle, m, k, n, flags_name):
    """Fused path (aligned, no split-K) and the two-kernel route it falls back to must both match
    matmul followed by bias_gelu on the CPU."""
    rng = np.random.default_rng(m + k + n)
    a = rng.standard_normal((m, k), dtype=np.float32)
    w = (0.05 * rng.standard_normal((k, n))).astype(np.float32)
    bias = (0.1 * rng.standard_normal(n)).astype(np.float32)
    H = oracle.HostTensor.from_array
    rpre = oracle.matmul(H(a), H(w))
    rout = oracle.bias_gelu(rpre, H(bias)).numpy()
    flags = F._lib.force_split_k(3) | F._lib.FORCE_TENSOR_PATH if flags_name == "split" else 0
    pre, out = F.matmul_bias_gelu(_dev(F, a), _dev(F, w), _dev(F, bias), flags=flags)
    F.device_status()
    bound = tol_3xtf32(k, a, w)
    assert float(np.max(np.abs(pre.numpy() - rpre.numpy()))) <= bound
    assert float(np.max(np.abs(out.numpy() - rout))) <= 1.2 * bound + 4e-6
    _, out_only = F.matmul_bias_gelu(_dev(F, a), _dev(F, w), _dev(F, bias), flags=flags, want_pre=False)
    F.device_status()
    assert np.array_equal(out_only.numpy(), out.numpy())


def test_batched_broadcast_weight_with_gelu(F, oracle):
    """Config 4's shape family at reduced size: [B, M, K] . [K, N] + b, GELU."""
    rng = np.random.default_rng(5)
    a = rng.standard_normal((3, 160, 96), dtype=np.float32)
    w = (0.02 * rng.standard_normal((96, 256))).astype(np.float32)
    bias = (0.02 * rng.standard_normal(256)).astype(np.float32)
    H = oracle.HostTensor.from_array
    rpre = oracle.matmul(H(a), H(w))
    rout = oracle.bias_gelu(rpre, H(bias)).numpy()
    pre, out = F.matmul_bias_gelu(_dev(F, a), _dev(F, w), _dev(F, bias))
    F.device_status()
    assert pre.shape == (3, 160, 256)
    assert float(np.max(np.abs(out.numpy() - rout))) <= 1.2 * tol_3xtf32(96, a, w) + 4e-6
