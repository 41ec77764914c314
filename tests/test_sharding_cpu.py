"""CPU: the multi-GPU sharding logic, run as world_size-2 gloo ranks with the CPU oracle standing in
for the GPU kernels.  Batch shards (broadcast weight) and row shards (2-D GEMM) must reproduce the
unsharded forward / input gradient exactly and the weight gradient after the reduce."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT
from framework_b200.sharding import DataParallelStep, panel_bounds, shard_bounds, shard_leading


def test_shard_bounds_cover_everything_once():
    for n in (0, 1, 7, 64, 8192):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
    assert shard_leading((64, 1024, 768), 3, 8) == (8, 1024, 768)
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def test_panel_bounds_are_aligned_and_cover_the_range():
    for n, panels, mult in ((8192, 4, 128), (1000, 4, 128), (100, 8, 128), (768, 3, 1), (5, 9, 1)):
        spans = panel_bounds(n, panels, mult)
        assert spans[0][0] == 0 and spans[-1][1] == n and len(spans) <= panels
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(lo % mult == 0 for lo, _ in spans) and all(hi > lo for lo, hi in spans)


def _worker(rank, world, port, a_shape, w_shape, q):
    """One rank: the step driver the GPU bench uses (DataParallelStep: forward, weight-gradient panels each
    reduced from one flat buffer, input gradient), with the CPU oracle standing in for the kernels."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle as O
    H = O.HostTensor
    rng = np.random.default_rng(0)
    a = rng.standard_normal(a_shape, dtype=np.float32)
    w = rng.standard_normal(w_shape, dtype=np.float32)
    bias = rng.standard_normal(w_shape[-1], dtype=np.float32)
    out_shape = a_shape[:-1] + (w_shape[-1],)
    dy = rng.standard_normal(out_shape, dtype=np.float32)
    lo, hi = shard_bounds(a_shape[0], rank, world)
    ha, hw, hdy = H.from_array(a[lo:hi]), H.from_array(w), H.from_array(dy[lo:hi])
    k, n = w_shape
    res = {}
    two_d = len(a_shape) == 2
    if two_d:      # row panels of dW: rows [p0, p1) need columns [p0, p1) of the shard's A
        spans = panel_bounds(k, 3, multiple=4)
        flat = torch.zeros(k * n)
        bufs = [flat[p0 * n:p1 * n] for p0, p1 in spans]

        def panel(p0, p1):
            _, dwp = O.matmul_backward(hdy, H.from_array(a[lo:hi, p0:p1]), H.from_array(w[p0:p1]), threads=1)
            flat[p0 * n:p1 * n] = torch.from_numpy(dwp.data)
        fns = [(lambda s=s: panel(*s)) for s in spans]
    else:          # dW and db side by side in one flat buffer: one collective call
        off = (k * n + 63) // 64 * 64
        flat = torch.zeros(off + n)
        bufs = [flat]

        def whole():
            _, dw = O.matmul_backward(hdy, ha, hw, threads=1)
            _, db = O.add_backward(hdy, hdy.shape, (n,), threads=1)
            flat[:k * n] = torch.from_numpy(dw.data)
            flat[off:] = torch.from_numpy(db.data)
        fns = [whole]

    def forward():
        res["y"] = O.add(O.matmul(ha, hw, threads=1), H.from_array(bias)).numpy()

    def input_grad():
        res["da"] = O.matmul_backward(hdy, ha, hw, threads=1)[0].numpy()

    step = DataParallelStep(forward, fns, bufs, input_grad, streams=None, dst=0)
    step()
    step.join()
    fa, fw, fdy = H.from_array(a), H.from_array(w), H.from_array(dy)
    full_y = O.add(O.matmul(fa, fw, threads=1), H.from_array(bias)).numpy()
    fda, fdw = O.matmul_backward(fdy, fa, fw, threads=1)
    ok = np.array_equal(res["y"], full_y[lo:hi]) and np.array_equal(res["da"], fda.numpy()[lo:hi])
    if rank == 0:
        kk = a_shape[0] * (a_shape[1] if len(a_shape) == 3 else 1)
        bound = 1e-5 * kk * float(np.abs(a).max()) * float(np.abs(dy).max())
        ok = ok and float(np.max(np.abs(flat[:k * n].numpy() - fdw.data))) <= bound
        if not two_d:
            _, fdb = O.add_backward(fdy, fdy.shape, (n,), threads=1)
            ok = ok and float(np.max(np.abs(flat[off:].numpy() - fdb.data))) <= 1e-5 * kk * float(np.abs(dy).max())
    q.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("a_shape,w_shape", [((6, 20, 12), (12, 16)), ((50, 24), (24, 10))])
def test_two_gloo_ranks_reproduce_the_unsharded_result(a_shape, w_shape):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, a_shape, w_shape, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == {0: True, 1: True}


def test_step_driver_reserves_sms_only_beside_a_reduce():
    """The driver asks for free SMs after it has issued a reduce and gives them back before the next first
    weight-gradient panel (or, with `reserve_forward` off, right after the input gradient).  Run without a
    process group: the collective is a no-op, the order of calls is what is checked."""
    if not torch.cuda.is_available():
        # streams=None path: no reservation is ever requested on the in-order path
        calls = []
        step = DataParallelStep(lambda: calls.append("fwd"), [lambda: calls.append("dW0"), lambda: calls.append("dW1")],
                                [torch.zeros(4), torch.zeros(4)], lambda: calls.append("dx"), streams=None,
                                reserve=lambda n: calls.append(("reserve", n)), reserve_sms=16)
        step()
        step.join()
        assert [c for c in calls if isinstance(c, str)] == ["fwd", "dW0", "dW1", "dx"]
        assert calls[-1] == ("reserve", 0)                    # join always hands the SMs back
        assert ("reserve", 16) not in calls
