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
from framework_b200.sharding import reduce_to_root, shard_bounds, shard_leading


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


def _worker(rank, world, port, a_shape, w_shape, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle as O
    rng = np.random.default_rng(0)
    a = rng.standard_normal(a_shape, dtype=np.float32)
    w = rng.standard_normal(w_shape, dtype=np.float32)
    out_shape = a_shape[:-1] + (w_shape[-1],)
    dy = rng.standard_normal(out_shape, dtype=np.float32)
    lo, hi = shard_bounds(a_shape[0], rank, world)
    ha, hw, hdy = (O.HostTensor.from_array(a[lo:hi]), O.HostTensor.from_array(w), O.HostTensor.from_array(dy[lo:hi]))
    y = O.matmul(ha, hw, threads=1).numpy()
    da, dw = O.matmul_backward(hdy, ha, hw, threads=1)
    flat = torch.from_numpy(dw.data.copy())
    reduce_to_root(flat, dst=0)
    full_y = O.matmul(O.HostTensor.from_array(a), O.HostTensor.from_array(w), threads=1).numpy()
    fda, fdw = O.matmul_backward(O.HostTensor.from_array(dy), O.HostTensor.from_array(a), O.HostTensor.from_array(w),
                                 threads=1)
    ok = np.array_equal(y, full_y[lo:hi]) and np.array_equal(da.numpy(), fda.numpy()[lo:hi])
    if rank == 0:
        k = a_shape[0] * (a_shape[1] if len(a_shape) == 3 else 1)
        bound = 1e-5 * k * float(np.abs(a).max()) * float(np.abs(dy).max())
        ok = ok and float(np.max(np.abs(flat.numpy() - fdw.data))) <= bound
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
