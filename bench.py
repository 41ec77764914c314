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


# --------------------------------------------------------------------------- workloads
class Workload:
    """Shapes and seeded synthetic inputs of one configuration.

    kind "gemm": y = a . b (+ bias); backward from dy gives da, db (, dbias).
    kind "attention": S = q . k^T (k^T a stride-only permute view), O = S . v; backward from dO
    gives dS, dV, dQ, dK^T -- the six GEMMs of the attention-shaped configuration.
    """

    def __init__(self, name, desc, a_shape, b_shape, *, bias=False, b_perm=None, dist_a="normal",
                 scale_b=1.0, kind="gemm"):
        self.name, self.desc, self.kind = name, desc, kind
        self.a_shape, self.b_shape = tuple(a_shape), tuple(b_shape)
        self.bias, self.b_perm = bias, b_perm
        self.dist_a, self.scale_b = dist_a, scale_b

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
    def batch(self):
        return int(np.prod(self.out_shape[:-2])) if len(self.out_shape) > 2 else 1

    @property
    def flops(self):
        """Algorithmic flops of forward + backward: 3 GEMMs of 2*M*N*K per batch (6 for attention)."""
        m, k, n = self.mkn
        one = 2 * m * n * k * self.batch
        return 6 * one if self.kind == "attention" else 3 * one

    @property
    def fwd_flops(self):
        return self.flops // 3

    def host_inputs(self, seed=0) -> dict:
        rng = np.random.default_rng(seed)

        def normal(shape, scale=1.0):
            return (scale * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
        if self.kind == "attention":
            return {"q": normal(self.a_shape), "k": normal(self.b_shape), "v": normal(self.a_shape),
                    "do": normal(self.a_shape)}
        a = rng.random(self.a_shape, dtype=np.float32) if self.dist_a == "uniform" else normal(self.a_shape)
        out = {"a": a, "b": normal(self.b_shape, self.scale_b)}
        if self.bias:
            out["bias"] = normal((self.mkn[2],), 0.02)
        out["dy"] = normal(self.out_shape)
        return out

    def with_a_shape(self, a_shape, note=""):
        b_shape = self.b_shape
        if self.kind == "attention" or (len(self.b_shape) == len(self.a_shape) and len(self.a_shape) > 2
                                        and self.b_shape[0] == self.a_shape[0]):
            b_shape = (a_shape[0],) + tuple(self.b_shape[1:])
        return Workload(self.name, self.desc + note, a_shape, b_shape, bias=self.bias, b_perm=self.b_perm,
                        dist_a=self.dist_a, scale_b=self.scale_b, kind=self.kind)


WORKLOADS = {
    "c1": Workload("c1", "2-D A[512,512].B[512,512] ~N(0,1)", (512, 512), (512, 512)),
    "c2": Workload("c2", "Linear step x[4096,1024].W[1024,4096]+b[4096], dy~N(0,1)", (4096, 1024), (1024, 4096),
                   bias=True, dist_a="uniform", scale_b=0.02),
    "c3": Workload("c3", "attention-shaped Q,K,V [8,12,512,64]: S=Q.K^T (K^T a permute view), O=S.V, fwd+bwd",
                   (8, 12, 512, 64), (8, 12, 512, 64), b_perm=(0, 1, 3, 2), kind="attention"),
    "c4": Workload("c4", "broadcast weight [64,1024,768].[768,3072], dW summed over the batch",
                   (64, 1024, 768), (768, 3072), scale_b=0.02),
    "c5a": Workload("c5a", "square 8192^3 ~N(0,1)", (8192, 8192), (8192, 8192)),
    "c5b1": Workload("c5b1", "skinny M=1, K=N=4096", (1, 4096), (4096, 4096)),
    "c5b4": Workload("c5b4", "skinny M=4, K=N=4096", (4, 4096), (4096, 4096)),
    "c5b16": Workload("c5b16", "skinny M=16, K=N=4096", (16, 4096), (4096, 4096)),
}
HBM_BOUND = ("c3", "c5b1", "c5b4", "c5b16")
# DRAM bytes per forward launch from ncu captures of the same launch
# (dram__bytes_read.sum + dram__bytes_write.sum; 3xTF32 build with CTA pairs).
NCU_TRAFFIC_BYTES = {"c2": 34.11e6 + 19.63e6}


def shard_workload(wl: Workload, rank: int, world: int) -> Workload:
    """Per-rank shard for the configurations that partition: batch shards for c4, row shards for
    c5a.  c2 is weak-scaled (every rank owns a full-size batch shard), the rest run as replicas."""
    if world == 1 or wl.name not in ("c4", "c5a"):
        return wl
    from framework_b200.sharding import shard_leading
    return wl.with_a_shape(shard_leading(wl.a_shape, rank, world), f" (1/{world} shard)")


class Problem:
    """Device-side instance of a workload: resident inputs, preallocated outputs, the call sequence."""

    def __init__(self, F, wl: Workload, host: dict, dev, flags: int):
        T = F.DeviceTensor
        self.F, self.wl, self.flags = F, wl, flags
        self.inp = {k: T.from_numpy(v, dev) for k, v in host.items()}
        if wl.kind == "attention":
            self.kt = self.inp["k"].permute(wl.b_perm)
            shp = wl.out_shape
            self.out = {"s": T.empty(shp, dev), "o": T.empty(wl.a_shape, dev), "ds": T.empty(shp, dev),
                        "dv": T.empty(wl.a_shape, dev), "dq": T.empty(wl.a_shape, dev),
                        "dkt": T.empty(self.kt.shape, dev)}
        else:
            self.b = self.inp["b"].permute(wl.b_perm) if wl.b_perm else self.inp["b"]
            self.out = {"y": T.empty(wl.out_shape, dev), "da": T.empty(wl.a_shape, dev),
                        "db": T.empty(self.b.shape, dev)}
            if wl.bias:
                self.out["dbias"] = T.empty((wl.mkn[2],), dev)

    def forward(self):
        F, i, o = self.F, self.inp, self.out
        if self.wl.kind == "attention":
            F.matmul(i["q"], self.kt, flags=self.flags, out=o["s"])
            F.matmul(o["s"], i["v"], flags=self.flags, out=o["o"])
        else:
            F.matmul(i["a"], self.b, i.get("bias"), flags=self.flags, out=o["y"])

    def backward(self):
        F, i, o = self.F, self.inp, self.out
        if self.wl.kind == "attention":
            F.matmul_backward(i["do"], o["s"], i["v"], flags=self.flags, da=o["ds"], db=o["dv"])
            F.matmul_backward(o["ds"], i["q"], self.kt, flags=self.flags, da=o["dq"], db=o["dkt"])
        else:
            F.matmul_backward(i["dy"], i["a"], self.b, flags=self.flags, da=o["da"], db=o["db"],
                              dbias=o.get("dbias"), want_dbias=self.wl.bias)

    def backward_weights(self):
        """dW (and db) only: what the data-parallel reduce needs first."""
        i, o = self.inp, self.out
        self.F.matmul_backward(i["dy"], i["a"], self.b, flags=self.flags, need_da=False, db=o["db"],
                               dbias=o.get("dbias"), want_dbias=self.wl.bias)

    def backward_inputs(self):
        i, o = self.inp, self.out
        self.F.matmul_backward(i["dy"], i["a"], self.b, flags=self.flags, da=o["da"], need_db=False)

    def weight_grads(self):
        return [self.out[k].storage for k in ("db", "dbias") if k in self.out]


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock, power and clock-event (throttle) reasons while the timed region runs.

    NVML is read directly from a thread every 2 ms (a timed region can be shorter than one `nvidia-smi -lms`
    period); `nvidia-smi` in a subprocess is the fallback when the NVML binding is missing.  Read-only queries.
    """
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []
        self.samples, self.smax, self._stop, self._thread, self.source = [], None, False, None, None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        index = self.gpu_index
        if visible:
            entry = visible.split(",")[self.gpu_index].strip()
            if entry.isdigit():
                index = int(entry)
            else:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(entry)
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)

    def start(self):
        try:
            nv, handle = self._nvml_handle()
            self.smax = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons

            def loop():
                while not self._stop:
                    try:
                        self.samples.append((time.time(), float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)),
                                             nv.nvmlDeviceGetPowerUsage(handle) / 1000.0, int(reasons_fn(handle))))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self.source = "nvml"
            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            return
        except Exception:
            self.source = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi"
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.source == "nvml":
            self._stop = True
            self._thread.join(timeout=1.0)
            rows = [r for r in self.samples if t0 <= r[0] <= t1] or self.samples[-3:]
            sm = [r[1] for r in rows]
            power = [r[2] for r in rows]
            mask = 0
            for r in rows:
                mask |= r[3]
            reasons = sorted(name for bit, name in self.REASON_BITS.items() if mask & bit)
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                    "sm_max_mhz": self.smax, "power_w_max": max(power) if power else None, "reasons": reasons,
                    "samples": len(sm), "source": "nvml, 2 ms period, timed region only"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        sm, power, smax, reasons = [], [], None, set()
        rows = [l for (t, l) in self.lines if t0 <= t <= t1 + 0.02] or [l for _, l in self.lines][-3:]
        for line in rows:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvidia-smi -lms 50"}


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    import framework_b200 as F
    from framework_b200.sharding import reduce_to_root

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    base = WORKLOADS[args.workload]
    wl = shard_workload(base, rank, world)
    flags = F._lib.PRECISION_TF32 if args.precision == "tf32" else 0
    host = wl.host_inputs(seed=rank)
    if world > 1 and wl.kind == "gemm":      # the weight (and bias) are replicated
        shared = wl.host_inputs(seed=0)
        for key in ("b", "bias"):
            if key in host:
                host[key] = shared[key]
    prob = Problem(F, wl, host, dev, flags)
    reduce_grads = world > 1 and wl.name in ("c2", "c4", "c5a")

    # Data parallel: the weight gradient is computed first and summed onto rank 0 on a second stream
    # while the input-gradient GEMM (and the next step's forward) run.
    comm = torch.cuda.Stream() if reduce_grads else None
    ev_w, ev_red = torch.cuda.Event(), torch.cuda.Event()

    def eager_step(pr=prob):
        pr.forward()
        if not reduce_grads:
            pr.backward()
            return
        main = torch.cuda.current_stream()
        main.wait_event(ev_red)              # the previous reduce is done with the gradient buffers
        pr.backward_weights()
        ev_w.record(main)
        with torch.cuda.stream(comm):
            comm.wait_event(ev_w)
            for g in pr.weight_grads():
                reduce_to_root(g, dst=0)
            ev_red.record(comm)
        pr.backward_inputs()

    def join_comm():
        if reduce_grads:
            torch.cuda.current_stream().wait_event(ev_red)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, after=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if after:
            after()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        eager_step()
    F.device_status()

    # Launch-bound workloads replay the step from a CUDA graph (same kernels, same order).
    step, graphed = eager_step, False
    est_ms = timed(eager_step, 5) / 5
    if world == 1 and args.graph != "off" and (args.graph == "on" or est_ms < 0.2):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            eager_step()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            eager_step()
        step, graphed = g.replay, True
        for _ in range(3):
            step()
        F.device_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    launches0 = F.launch_count()
    eager_step()
    launches_per_step = F.launch_count() - launches0
    torch.cuda.synchronize()
    t_wall0 = time.time()
    total_ms = timed(step, args.steps, after=join_comm)
    t_wall1 = time.time()
    F.device_status()
    ms_per_step = total_ms / args.steps
    value = wl.flops * world / (ms_per_step * 1e-3) / 1e12
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    # ---- roofline of the dominant kernel: the forward launch(es) timed alone ----
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    # The forward launch is timed alone, against the burst peak: let the power state of the timed region
    # above (which ends at the power cap) settle first.
    torch.cuda.synchronize()
    time.sleep(0.5)
    l0 = F.launch_count()
    prob.forward()
    fwd_launches = F.launch_count() - l0
    fwd_steps = min(args.steps, 50)
    fwd_ms = timed(prob.forward, fwd_steps) / fwd_steps
    if wl.name in HBM_BOUND:
        if wl.kind == "attention":   # S written and read once, Q, K, V read, O written
            alg_bytes = 4.0 * (2 * np.prod(wl.out_shape) + 4 * np.prod(wl.a_shape))
        else:                        # each operand read once, the output written once
            alg_bytes = 4.0 * (np.prod(wl.a_shape) + np.prod(wl.b_shape) + np.prod(wl.out_shape))
        peak = peaks.get("hbm_gbs", 6650.0)
        achieved = alg_bytes / (fwd_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": None, "kernel": "forward call(s): " + ("gemm_tc_kernel x2" if wl.kind == "attention"
                                                                      else "skinny_fwd_kernel + reduce"),
                    "launches_per_call": fwd_launches, "algorithmic_bytes": alg_bytes,
                    "peak_source": "measured hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650"}
    else:
        bf16 = peaks.get("bf16_tflops", 1590.0)
        peak = bf16 / 2.0
        achieved = wl.fwd_flops / (fwd_ms * 1e-3) / 1e12
        issued = achieved * (1 if args.precision == "tf32" else 3)
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": NCU_TRAFFIC_BYTES.get(wl.name) if args.precision != "tf32" else None,
                    "traffic_unit": "bytes per launch (ncu dram read+write)",
                    "algorithmic_bytes": 4.0 * (np.prod(wl.a_shape) + np.prod(wl.b_shape) + np.prod(wl.out_shape)),
                    "kernel": "gemm_tc_kernel (forward GEMM launch, bias fused)",
                    "issued_tflops": issued, "issued_frac": issued / peak,
                    "note": ("3xTF32 issues 3 MMAs per product: algorithmic ceiling = peak/3"
                             if args.precision != "tf32" else "single-pass TF32"),
                    "peak_source": ("measured bf16_tflops/2 (no TF32 figure in MEASURED_PEAKS.json)"
                                    if "bf16_tflops" in peaks else "fallback 1590/2")}

    # ---- end to end: pinned host buffers -> device -> C ABI -> host buffers ------------------
    # Three streams: uploads, the C-ABI calls, downloads.  Inputs and outputs are double buffered on the
    # device so that step i+1's upload and step i-1's download overlap step i's kernels; every step still
    # moves all of its inputs in and all of its outputs out.
    h_in = {k: torch.from_numpy(np.ascontiguousarray(v).reshape(-1)).pin_memory() for k, v in host.items()}
    h_out = {k: torch.empty(t.size, dtype=torch.float32).pin_memory() for k, t in prob.out.items()}
    h2d = sum(h.numel() * 4 for h in h_in.values())
    d2h = sum(h.numel() * 4 for h in h_out.values())
    s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    slots = [prob, Problem(F, wl, host, dev, flags)]
    ev_in = [torch.cuda.Event() for _ in slots]
    ev_done = [torch.cuda.Event() for _ in slots]
    ev_out = [torch.cuda.Event() for _ in slots]
    counter = [0]

    def e2e_step():
        i = counter[0] % len(slots)
        counter[0] += 1
        pr = slots[i]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[i])          # the kernels that last read this slot's inputs are done
            for key, h in h_in.items():
                pr.inp[key].storage[: h.numel()].copy_(h, non_blocking=True)
            ev_in[i].record(s_in)
        s_main.wait_event(ev_in[i])
        s_main.wait_event(ev_out[i])             # the download that last read this slot's outputs is done
        eager_step(pr)
        join_comm()
        ev_done[i].record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[i])
            for key, h in h_out.items():
                t = pr.out[key]
                h.copy_(t.storage[: t.size], non_blocking=True)
            ev_out[i].record(s_out)

    def e2e_join():
        join_comm()
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    for _ in range(3):
        e2e_step()
    e2e_join()
    torch.cuda.synchronize()
    e2e_steps = max(4, min(args.steps, 50))
    e2e_ms = timed(e2e_step, e2e_steps, after=e2e_join) / e2e_steps
    e2e_value = wl.flops * world / (e2e_ms * 1e-3) / 1e12
    F.device_status()

    # Last measurement of the run (it heats the GPU to its power cap).  NVML refreshes its clock and throttle readings far more slowly than a timed region of ~0.1 s lasts, so
    # the same steps are repeated, untimed, for about a second with a second sampler: what the clocks settle
    # at under this workload, reported beside the readings taken during the timed region.
    sustain_steps = int(min(20000, max(args.steps, 1000.0 / max(ms_per_step, 1e-3))))
    sustain = ClockSampler(local_rank)
    if rank == 0:
        sustain.start()
    t_s0 = time.time()
    sustain_ms = timed(step, sustain_steps, after=join_comm)
    t_s1 = time.time()
    if rank == 0:
        settled = sustain.stop(t_s0 + 0.5 * (t_s1 - t_s0), t_s1)       # second half of the window
        clocks["sustained"] = {"seconds": round(t_s1 - t_s0, 2), "steps": sustain_steps,
                               "ms_per_step": sustain_ms / sustain_steps, "sm_mhz": settled.get("sm_mhz"),
                               "sm_min_mhz": settled.get("sm_min_mhz"), "power_w_max": settled.get("power_w_max"),
                               "reasons": settled.get("reasons"), "samples": settled.get("samples")}
        for r in settled.get("reasons") or []:
            if r not in clocks["reasons"]:
                clocks["reasons"].append(r)

    if rank == 0:
        cpu = cpu_baseline_sample(base, threads=1) if (world == 1 and not args.no_cpu) else None
        ws = working_set_mb(wl)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if base.name in ("c4", "c5a") else "weak", "vs_baseline": None,
            "dtype": "f32 storage, 3xTF32 tensor-core arithmetic (f32 accumulate)" if args.precision != "tf32"
                     else "f32 storage, single-pass TF32 arithmetic (reduced precision mode)",
            "data": "synthetic (seeded numpy default_rng: x~U[0,1), W~N(0,0.02), b~N(0,0.02), dy~N(0,1))"
                    if wl.name == "c2" else "synthetic (seeded numpy default_rng, ~N(0,1))",
            "config": {"workload": f"{base.name}: {base.desc}", "per_gpu": f"{wl.a_shape} x {wl.b_logical}",
                       "parallelism": "single GPU" if world == 1 else
                                      f"dp{world}: batch shard per rank" + (", NCCL reduce of dW" + ("+db" if wl.bias else "") + " overlapped with the dx GEMM"
                                                                            if reduce_grads else ", replicas"),
                       "precision": args.precision, "cuda_graph": graphed,
                       "l2": (f"working set {ws:.0f} MB per step vs 126 MB L2, no flush" if ws > 126 else
                              f"working set {ws:.0f} MB fits the 126 MB L2; not flushed between steps (stated)"),
                       "flops_per_step_per_gpu": wl.flops},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "overlap": "3 streams, 2 device slots"},
            "gpu_launches": int(launches_per_step * args.steps),
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
    if wl.kind == "attention":
        elems = 2 * np.prod(wl.out_shape) + 8 * np.prod(wl.a_shape)
    else:
        elems = 2 * np.prod(wl.a_shape) + 2 * np.prod(wl.b_shape) + 2 * np.prod(wl.out_shape)
    return float(elems) * 4 / 1e6


# --------------------------------------------------------------------------- CPU arm
def cpu_tensors(O, wl: Workload) -> dict:
    host = wl.host_inputs(seed=0)
    t = {k: O.HostTensor.from_array(v) for k, v in host.items()}
    if wl.kind == "attention":
        t["kt"] = O.permute(t["k"], wl.b_perm)
    elif wl.b_perm:
        t["b"] = O.permute(t["b"], wl.b_perm)
    return t


def cpu_step(O, wl: Workload, t: dict, threads: int):
    """The reference CPU backend's call sequence for one fwd+bwd step (oracle port)."""
    if wl.kind == "attention":
        s = O.matmul(t["q"], t["kt"], threads=threads)
        O.matmul(s, t["v"], threads=threads)
        ds, _ = O.matmul_backward(t["do"], s, t["v"], threads=threads)
        return O.matmul_backward(ds, t["q"], t["kt"], threads=threads)
    y = O.matmul(t["a"], t["b"], threads=threads)                              # ops/matmul.rs:19-78
    dy = t["dy"]
    if "bias" in t:
        y = O.add(y, t["bias"])                                                # ops/elementwise.rs:62-73
        dy, _ = O.add_backward(dy, y.shape, t["bias"].shape, threads=threads)  # :199-211
    return O.matmul_backward(dy, t["a"], t["b"], threads=threads)              # ops/matmul.rs:200-222


def cpu_sample_workload(wl: Workload, budget_gflop: float):
    """Bounds the CPU work: whole step if it fits the budget, else a leading slice of the batch / rows."""
    if wl.flops / 1e9 <= budget_gflop:
        return wl, "whole step"
    lead = wl.a_shape[0]
    keep = max(1, int(lead * budget_gflop * 1e9 / wl.flops))
    small = wl.with_a_shape((keep,) + tuple(wl.a_shape[1:]))
    return small, f"leading {keep}/{lead} of the first dim of A (same K, N)"


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline_sample(wl: Workload, threads: int) -> dict:
    import oracle as O
    O.build()
    small, what = cpu_sample_workload(wl, budget_gflop=120.0 * max(threads, 1))
    tens = cpu_tensors(O, small)
    t0 = time.perf_counter()
    cpu_step(O, small, tens, threads)
    dt = time.perf_counter() - t0
    return {"value": small.flops / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{what}; {small.flops / 1e9:.1f} GFLOP in {dt:.2f} s; C restatement of the reference's "
                      f"single-threaded CPU backend (gcc -O3 -ffp-contract=off)",
            "host_cores": host_threads()}


def run_reference(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as O
    O.build()
    threads = host_threads()      # not OMP_NUM_THREADS: launchers set that to 1
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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--precision", default="3xtf32", choices=["3xtf32", "tf32"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the step from a CUDA graph (auto: only for steps under 0.2 ms)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
