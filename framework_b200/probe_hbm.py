"""Times the HBM-bound kernels of the library on inputs larger than L2 and prints achieved GB/s.

``python -m framework_b200.probe_hbm [--iters N] [--only softmax,adamw,skinny]``

Algorithmic bytes: softmax forward 8 B/element (read x, write out), backward 12 B/element; gradient sum of
squares 4 B/element; AdamW step 28 B/element (32 with the clipped gradient written back); skinny products
one pass over the weight.  Timing is CUDA events around a CUDA-graph replay of ``iters`` back-to-back calls after 3 warm-up calls.
The same command under ``ncu -k regex:...`` gives the per-kernel DRAM counters.
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

import framework_b200 as F
from framework_b200 import ops


def _tensor(*shape) -> F.DeviceTensor:
    return F.DeviceTensor(torch.randn(int(np.prod(shape)), device="cuda"), shape)


def _time(fn, iters: int) -> float:
    """Seconds per call: `iters` calls captured into one CUDA graph and replayed, so that launch latency of the
    host interpreter does not hide a 10 us kernel."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(iters):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters * 1e-3


def _report(name: str, nbytes: float, seconds: float) -> None:
    print(f"{name:44s} {seconds * 1e6:9.1f} us  {nbytes / seconds / 1e9:8.1f} GB/s", flush=True)


def probe_softmax(iters: int) -> None:
    for shape in ((8, 12, 512, 512), (64, 12, 512, 512)):
        x, g = _tensor(*shape), _tensor(*shape)
        sm = F.softmax(x, -1)
        _report(f"softmax fwd {shape}", 8.0 * x.size, _time(lambda: F.softmax(x, -1), iters))
        _report(f"softmax bwd {shape}", 12.0 * x.size, _time(lambda: F.softmax_backward(g, sm, -1), iters))


def probe_adamw(iters: int) -> None:
    n = 64 * 1024 * 1024
    p, m, v, g = (_tensor(n) for _ in range(4))
    v.storage.abs_()
    _report(f"grad_sumsq n={n}", 4.0 * n, _time(lambda: ops._grad_sumsq([g]), iters))
    _report(f"adamw_step n={n}", 28.0 * n,
            _time(lambda: F.adamw_step(p, m, v, g, lr=1e-3, step=3, weight_decay=0.01), iters))
    sumsq = ops._grad_sumsq([g])
    _report(f"adamw_step + clip n={n}", 32.0 * n,
            _time(lambda: F.adamw_step(p, m, v, g, lr=1e-3, step=3, weight_decay=0.01, grad_sumsq=sumsq,
                                       max_grad_norm=1.0), iters))


def probe_skinny(iters: int) -> None:
    """Three weights (201 MB) are used in turn, so that no call finds its 67 MB weight in the 126 MB L2."""
    k = n = 4096
    ws = [_tensor(k, n) for _ in range(3)]
    dws = [F.DeviceTensor.empty((k, n)) for _ in range(3)]
    turn = [0]

    def nxt():
        turn[0] = (turn[0] + 1) % 3
        return turn[0]

    for m in (1, 4):
        x, dy = _tensor(m, k), _tensor(m, n)
        y, dx = F.DeviceTensor.empty((m, n)), F.DeviceTensor.empty((m, k))
        _report(f"skinny fwd M={m} K=N=4096", 4.0 * k * n, _time(lambda: F.matmul(x, ws[nxt()], out=y), iters))
        _report(f"skinny dx  M={m}", 4.0 * k * n,
                _time(lambda: F.matmul_backward(dy, x, ws[nxt()], da=dx, need_db=False), iters))
        _report(f"skinny dW  M={m}", 4.0 * k * n,
                _time(lambda: F.matmul_backward(dy, x, ws[0], db=dws[nxt()], need_da=False), iters))
    x, y = _tensor(8, k), F.DeviceTensor.empty((8, n))
    _report("skinny fwd M=8 K=N=4096", 4.0 * k * n, _time(lambda: F.matmul(x, ws[nxt()], out=y), iters))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="softmax,adamw,skinny")
    args = ap.parse_args()
    which = set(args.only.split(","))
    if "softmax" in which:
        probe_softmax(args.iters)
    if "adamw" in which:
        probe_adamw(args.iters)
    if "skinny" in which:
        probe_skinny(args.iters)
    print("device status", F.device_status())


if __name__ == "__main__":
    main()
