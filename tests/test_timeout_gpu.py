"""GPU: the bounded device-side waits, made to run out.

Every wait of the tensor-core kernel (mbarrier phases, flags of the balanced tail) has a limit in clock
cycles; when it runs out the waiter records a role/slot code in a device word, raises the CTA's abort flag,
all roles drain to the common exit (copies in flight are awaited with their own limit, tensor memory is
freed) and the kernel RETURNS -- nothing traps, the context stays usable.  The reference has no counterpart
(it unwraps, ops/matmul.rs:172).  Here the limit is shortened to about a millisecond through the
environment and a test hook makes the TMA producer arm one pipeline stage without issuing its copies, so the
stage never fills: the waiters give up, `mni_b200_device_status` reports MNI_B200_ERR_TIMEOUT with the
recorded word, and the next, ordinary product on the same device is correct and leaves the status clean."""
import numpy as np
import pytest

from conftest import tol_3xtf32

pytestmark = pytest.mark.gpu

SHORT_LIMIT = "2000000"          # clock cycles: about 1 ms


@pytest.mark.parametrize("variant,env,flags", [
    ("cta_pair_256", {"MNI_B200_BN": "256"}, 0),
    ("lone_cta_tensor_memory_a", {"MNI_B200_BN": "64"}, 0),
    ("lone_cta_single_pass", {"MNI_B200_BN": "128"}, 1),
])
def test_wait_limit_runs_out_then_the_library_recovers(F, oracle, monkeypatch, variant, env, flags):
    rng = np.random.default_rng(5)
    a = rng.standard_normal((512, 512), dtype=np.float32)
    b = rng.standard_normal((512, 512), dtype=np.float32)
    ad, bd = F.DeviceTensor.from_numpy(a), F.DeviceTensor.from_numpy(b)
    F.device_status()                                    # clean before
    for key, val in env.items():
        monkeypatch.setenv(key, val)
    monkeypatch.setenv("MNI_B200_WAIT_CYCLES", SHORT_LIMIT)
    monkeypatch.setenv("MNI_B200_TEST_WITHHOLD_KBLOCK", "3")
    F.matmul(ad, bd, flags=F._lib.FORCE_TENSOR_PATH | flags)        # returns: the launch itself succeeds
    with pytest.raises(F._lib.MniError) as ei:
        F.device_status()
    assert ei.value.status == 8, ei.value                           # MNI_B200_ERR_TIMEOUT
    assert "bounded wait" in ei.value.message and "role" in ei.value.message
    monkeypatch.delenv("MNI_B200_TEST_WITHHOLD_KBLOCK")
    monkeypatch.delenv("MNI_B200_WAIT_CYCLES")
    assert F.device_status() == 0                                   # the record was cleared by the read
    out = F.matmul(ad, bd, flags=F._lib.FORCE_TENSOR_PATH | flags)
    assert F.device_status() == 0
    ref = oracle.matmul(oracle.HostTensor.from_array(a), oracle.HostTensor.from_array(b)).numpy()
    if flags & 1:
        assert np.linalg.norm(out.numpy() - ref) <= 2e-3 * np.linalg.norm(ref)
    else:
        assert float(np.max(np.abs(out.numpy() - ref))) <= tol_3xtf32(512, a, b)


def test_withhold_hook_is_ignored_without_a_short_limit(F, oracle, monkeypatch):
    """The hook only acts together with a shortened limit, so a stray environment variable cannot stall a
    production run for the default limit of about two seconds."""
    monkeypatch.setenv("MNI_B200_TEST_WITHHOLD_KBLOCK", "2")
    rng = np.random.default_rng(6)
    a = rng.standard_normal((256, 256), dtype=np.float32)
    b = rng.standard_normal((256, 256), dtype=np.float32)
    out = F.matmul(F.DeviceTensor.from_numpy(a), F.DeviceTensor.from_numpy(b), flags=F._lib.FORCE_TENSOR_PATH)
    assert F.device_status() == 0
    ref = oracle.matmul(oracle.HostTensor.from_array(a), oracle.HostTensor.from_array(b)).numpy()
    assert float(np.max(np.abs(out.numpy() - ref))) <= tol_3xtf32(256, a, b)
