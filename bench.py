#!/usr/bin/env python
"""Benchmark of the matmul hot path: f32 matmul forward+backward TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One "step" is one forward+backward pass of the workload through the C ABI of
libmni_b200.so.  The default workload is the Linear-layer training step
(x[4096,1024] . W[1024,4096] + b, backward with dy ~N(0,1) giving dx, dW, db).  With
N > 1 every rank runs the step on its own batch shard and the weight and bias
gradients are summed onto rank 0 with an NCCL reduce (data parallel, weak scaling).

The JSON line carries: `value` (device-resident inputs, CUDA-event timing, max over
ranks), `e2e` (pinned host buffers in, host buffers out, copies inside the timed
region), `roofline` of the dominant kernel, and `cpu_baseline` (the CPU oracle, a
restatement of the reference's single-threaded CPU backend, timed on this host).
`--impl reference` times that CPU implementation alone, on all host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "f32_matmul_fwd_bwd_tflops"
UNIT = "TFLOP/s"
L2_BYTES = 126 * 1024 * 1024


# --------------------------------------------------------------------------- workloads
class Workload:
    """Shapes, seeded synthetic inputs and the fwd+bwd call sequence of one configuration."""

    def __init__(self, name, desc, a_shape, b_shape, *, bias=False, b_perm=None, dist_a="normal",
                 dist_b="normal", scale_b=1.0):
        self.name, self.desc = name, desc
        self.a_shape, self.b_shape = tuple(a_shape), tuple(b_shape)
        self.bias, self.b_perm = bias, b_perm
        self.dist_a, self.dist_b, self.scale_b = dist_a, dist_b, scale_b

    # logical shapes ----------------------------------------------------------
    @property
    def b_logical(self):
        return tuple(self.b_shape[d] for d in self.b_perm) if self.b_perm else self.b_shape

    @property
    def mkn(self):
        return self.a_shape[-2], self.a_shape[-1], self.b_logical[-1]

    @property
    def out_shape(self):
        from framework_b200.ops import broadcast_shape
        m, _, n = self.mkn
        return broadcast_shape(self.a_shape[:-2], self.b_logical[:-2]) + (m, n)

    @property
    def flops(self):
        """Algorithmic flops of forward + backward = 3 GEMMs of 2*M*N*K per output batch."""
        m, k, n = self.mkn
        batch = int(np.prod(self.out_shape[:-2])) if len(self.out_shape) > 2 else 1
        return 3 * 2 * m * n * k * batch

    def host_inputs(self, seed=0):
        rng = np.random.default_rng(seed)

        def draw(shape, dist, scale):
            if dist == "uniform":
                return rng.random(shape, dtype=np.float32)
            return (scale * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
        a = draw(self.a_shape, self.dist_a, 1.0)
        b = draw(self.b_shape, self.dist_b, self.scale_b)
        bias = draw((self.mkn[2],), "normal", 0.02) if self.bias else None
        dy = draw(self.out_shape, "normal", 1.0)
        return a, b, bias, dy


WORKLOADS = {
    "c1": Workload("c1", "2-D A[512,512].B[512,512] ~N(0,1)", (512, 512), (512, 512)),
    "c2": Workload("c2", "Linear step x[4096,1024].W[1024,4096]+b[4096], dy~N(0,1)", (4096, 1024), (1024, 4096),
                   bias=True, dist_a="uniform", scale_b=0.02),
    "c3": Workload("c3", "attention-shaped Q.K^T, K^T a permute(0,1,3,2) view of [8,12,512,64]",
                   (8, 12, 512, 64), (8, 12, 512, 64), b_perm=(0, 1, 3, 2)),
    "c4": Workload("c4", "broadcast weight [64,1024,768].[768,3072], dW summed over the batch",
                   (64, 1024, 768), (768, 3072), scale_b=0.02),
    "c5a": Workload("c5a", "square 8192^3 ~N(0,1)", (8192, 8192), (8192, 8192)),
    "c5b1": Workload("c5b1", "skinny M=1, K=N=4096", (1, 4096), (4096, 4096)),
    "c5b4": Workload("c5b4", "skinny M=4, K=N=4096", (4, 4096), (4096, 4096)),
    "c5b16": Workload("c5b16", "skinny M=16, K=N=4096", (16, 4096), (4096, 4096)),
}


def shard_workload(wl: Workload, world: int) -> Workload:
    """Per-rank shard for the configurations that partition: batch shards for c4, row shards for
    c5a.  c2 is weak-scaled (every rank owns a full-size batch shard), the rest run as replicas."""
    if world == 1 or wl.name not in ("c4", "c5a"):
        return wl
    from framework_b200.sharding import shard_leading
    a_shape = shard_leading(wl.a_shape, int(os.environ.get("RANK", "0")), world)
    return Workload(wl.name, wl.desc + f" (1/{world} shard)", a_shape, wl.b_shape, bias=wl.bias,
                    b_perm=wl.b_perm, dist_a=wl.dist_a, dist_b=wl.dist_b, scale_b=wl.scale_b)


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        rows = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for _, l in self.lines]
        for line in rows:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    import framework_b200 as F
    from framework_b200.sharding import reduce_to_root

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    base = WORKLOADS[args.workload]
    wl = shard_workload(base, world)
    flags = F._lib.PRECISION_TF32 if args.precision == "tf32" else 0
    a_np, b_np, bias_np, dy_np = wl.host_inputs(seed=rank)
    if world > 1:   # the weight (and bias) are replicated
        _, b_np, bias_np, _ = wl.host_inputs(seed=0)
    T = F.DeviceTensor

    def to_dev(x):
        return T.from_numpy(x, dev) if x is not None else None
    a, b, bias, dy = to_dev(a_np), to_dev(b_np), to_dev(bias_np), to_dev(dy_np)
    if wl.b_perm:
        b = b.permute(wl.b_perm)
    y = T.empty(wl.out_shape, dev)
    da, db = T.empty(a.shape, dev), T.empty(b.shape, dev)
    dbias = T.empty((wl.mkn[2],), dev) if wl.bias else None
    reduce_grads = world > 1 and wl.name in ("c2", "c4", "c5a")

    def step():
        F.matmul(a, b, bias, flags=flags, out=y)
        F.matmul_backward(dy, a, b, flags=flags, da=da, db=db, dbias=dbias, want_dbias=wl.bias)
        if reduce_grads:
            reduce_to_root(db.storage, dst=0)
            if dbias is not None:
                reduce_to_root(dbias.storage, dst=0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step()
    F.device_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    t_wall0 = time.time()
    launches0 = F.launch_count()
    total_ms = timed(step, args.steps)
    launches = F.launch_count() - launches0
    t_wall1 = time.time()
    F.device_status()
    ms_per_step = total_ms / args.steps
    value = wl.flops * world / (ms_per_step * 1e-3) / 1e12

    # ---- roofline of the dominant kernel (the tensor-core GEMM; the skinny kernels for c5b) ----
    m, k, n = wl.mkn
    batch = int(np.prod(wl.out_shape[:-2])) if len(wl.out_shape) > 2 else 1
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass

    def fwd_only():
        F.matmul(a, b, bias, flags=flags, out=y)
    torch.cuda.synchronize()
    l0 = F.launch_count()
    fwd_ms = timed(fwd_only, args.steps) / args.steps
    fwd_launches = (F.launch_count() - l0) // args.steps
    skinny = wl.name.startswith("c5b") or wl.name == "c3"
    if skinny:
        # HBM-bound shapes: each operand read once, the output written once.
        alg_bytes = 4.0 * (np.prod(a.shape) + np.prod(b.shape) + np.prod(wl.out_shape))
        peak = peaks.get("hbm_gbs", 6650.0)
        achieved = alg_bytes / (fwd_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": None, "kernel": "forward call", "launches_per_call": fwd_launches,
                    "peak_source": "measured hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650"}
    else:
        alg = 2.0 * m * n * k * batch
        bf16 = peaks.get("bf16_tflops", 1590.0)
        peak = bf16 / 2.0
        achieved = alg / (fwd_ms * 1e-3) / 1e12
        issued = achieved * (1 if args.precision == "tf32" else 3)
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": None, "kernel": "gemm_tc_kernel (forward GEMM launch, bias fused)",
                    "issued_tflops": issued, "issued_frac": issued / peak,
                    "note": "3xTF32 issues 3 MMAs per product: algorithmic ceiling = peak/3" if args.precision != "tf32" else "single-pass TF32",
                    "peak_source": ("measured bf16_tflops/2 (no TF32 figure in MEASURED_PEAKS.json)"
                                    if "bf16_tflops" in peaks else "fallback 1590/2")}

    # ---- end to end: pinned host buffers -> device -> C ABI -> host buffers ------------------
    def pin(x):
        return torch.from_numpy(np.ascontiguousarray(x).reshape(-1)).pin_memory() if x is not None else None
    h_in = [pin(x) for x in (a_np, b_np, bias_np, dy_np)]
    d_in = [t.storage if t is not None else None for t in (a, b, bias, dy)]
    outs = [t for t in (y, da, db, dbias) if t is not None]
    h_out = [torch.empty(t.size, dtype=torch.float32).pin_memory() for t in outs]
    h2d = sum(h.numel() * 4 for h in h_in if h is not None)
    d2h = sum(h.numel() * 4 for h in h_out)

    def e2e_step():
        for h, d in zip(h_in, d_in):
            if h is not None:
                d[: h.numel()].copy_(h, non_blocking=True)
        step()
        for h, t in zip(h_out, outs):
            h.copy_(t.storage[: t.size], non_blocking=True)

    for _ in range(2):
        e2e_step()
    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms = timed(e2e_step, e2e_steps) / e2e_steps
    e2e_value = wl.flops * world / (e2e_ms * 1e-3) / 1e12
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None

    if rank == 0:
        cpu = cpu_baseline_sample(base, threads=1) if (world == 1 and not args.no_cpu) else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 storage, 3xTF32 tensor-core arithmetic (f32 accumulate)" if args.precision != "tf32"
                     else "f32 storage, single-pass TF32 arithmetic (reduced precision mode)",
            "data": "synthetic (seeded numpy default_rng: x~U[0,1), W~N(0,0.02), b~N(0,0.02), dy~N(0,1))"
                    if wl.name == "c2" else "synthetic (seeded numpy default_rng)",
            "config": {"workload": f"{base.name}: {base.desc}", "per_gpu": f"{wl.a_shape} x {wl.b_logical}",
                       "parallelism": "single GPU" if world == 1 else
                                      f"dp{world}: batch shard per rank, NCCL reduce of dW" + ("+db" if wl.bias else ""),
                       "precision": args.precision,
                       "l2": f"working set {working_set_mb(wl):.0f} MB per step vs 126 MB L2, no flush"
                             if working_set_mb(wl) > 126 else "working set fits L2; buffers not flushed (stated)",
                       "flops_per_step_per_gpu": wl.flops},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": roofline,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def working_set_mb(wl: Workload) -> float:
    elems = 2 * np.prod(wl.a_shape) + 2 * np.prod(wl.b_shape) + 2 * np.prod(wl.out_shape)
    return float(elems) * 4 / 1e6


# --------------------------------------------------------------------------- CPU arm
def cpu_step(O, wl: Workload, tensors, threads: int):
    """The reference CPU backend's call sequence for one fwd+bwd step (oracle port)."""
    a, b, bias, dy = tensors
    y = O.matmul(a, b, threads=threads)                                    # ops/matmul.rs:19-78
    if bias is not None:
        y = O.add(y, bias)                                                 # ops/elementwise.rs:62-73
        dy_in, _ = O.add_backward(dy, y.shape, bias.shape, threads=threads)  # :199-211
    else:
        dy_in = dy
    return O.matmul_backward(dy_in, a, b, threads=threads)                 # ops/matmul.rs:200-222


def cpu_tensors(O, wl: Workload):
    a_np, b_np, bias_np, dy_np = wl.host_inputs(seed=0)
    a, b = O.HostTensor.from_array(a_np), O.HostTensor.from_array(b_np)
    if wl.b_perm:
        b = O.permute(b, wl.b_perm)
    bias = O.HostTensor.from_array(bias_np) if bias_np is not None else None
    return a, b, bias, O.HostTensor.from_array(dy_np)


def cpu_sample_workload(wl: Workload, budget_gflop: float) -> (Workload, str):
    """Bounds the CPU work: whole step if it fits the budget, else a leading slice of the batch / rows."""
    if wl.flops / 1e9 <= budget_gflop:
        return wl, "whole step"
    frac = budget_gflop * 1e9 / wl.flops
    a_shape = list(wl.a_shape)
    lead = a_shape[0]
    keep = max(1, int(lead * frac))
    a_shape[0] = keep
    if len(wl.b_shape) == len(wl.a_shape) and wl.b_shape[0] == lead and len(wl.a_shape) > 2:
        b_shape = list(wl.b_shape)
        b_shape[0] = keep
    else:
        b_shape = wl.b_shape
    small = Workload(wl.name, wl.desc, a_shape, b_shape, bias=wl.bias, b_perm=wl.b_perm, dist_a=wl.dist_a,
                     dist_b=wl.dist_b, scale_b=wl.scale_b)
    return small, f"leading {keep}/{lead} of the first dim of A (same K, N)"


def cpu_baseline_sample(wl: Workload, threads: int) -> dict:
    import oracle as O
    O.build()
    per_core = 6.0  # GFLOP/s order of magnitude of the scalar loop; only sizes the sample
    small, what = cpu_sample_workload(wl, budget_gflop=20.0 * per_core * max(threads, 1))
    tens = cpu_tensors(O, small)
    t0 = time.perf_counter()
    cpu_step(O, small, tens, threads)
    dt = time.perf_counter() - t0
    return {"value": small.flops / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{what}; {small.flops / 1e9:.1f} GFLOP in {dt:.2f} s; C restatement of the reference's "
                      f"single-threaded CPU backend (gcc -O3 -ffp-contract=off)",
            "host_cores": os.cpu_count()}


def run_reference(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as O
    O.build()
    threads = O.max_threads()
    wl = WORKLOADS[args.workload]
    small, what = cpu_sample_workload(wl, budget_gflop=14.0 * threads)
    tens = cpu_tensors(O, small)
    warm = min(args.warmup, 1)
    for _ in range(warm):
        cpu_step(O, small, tens, threads)
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(O, small, tens, threads)
    dt = (time.perf_counter() - t0) / steps
    value = small.flops / dt / 1e12
    sample = (f"{what}; {small.flops / 1e9:.1f} GFLOP per step, {steps} timed steps; the reference's CPU backend is "
              f"single-threaded, this run spreads its row loop over {threads} threads (bit-identical results)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic (seeded numpy default_rng)",
        "config": {"workload": f"{wl.name}: {wl.desc}", "parallelism": f"CPU, {threads} threads"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--precision", default="3xtf32", choices=["3xtf32", "tf32"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
