#!/usr/bin/env python
"""Benchmark of the matmul hot path: f32 matmul forward+backward TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--impl reference]

One "step" is one forward+backward pass of the workload through the C ABI of
libmni_b200.so.  The default workload is the broadcast-weight GEMM
(activations [64,1024,768] . weight [768,3072], backward summing dW over the batch), the
configuration that shards: with N > 1 the 64 batches are split over the ranks (strong
scaling, one rank per GPU), every rank runs forward, dW and dA on its shard, and dW is
summed onto rank 0 with one NCCL reduce that overlaps the dA GEMM.  `--workload c5a` shards
the 8192^3 square by rows of A and reduces dB in row panels as they complete; `--workload c2`
is the Linear training step, weak-scaled; c1 / c3 / c5b* run as replicas; `softmax` and
`adamw` time the pointwise neighbours of the path in GB/s.

The JSON line carries: `value` (device-resident inputs, CUDA-event timing, max over
ranks), `e2e` (pinned host buffers in, host buffers out, copies inside the timed
region), `roofline` of the dominant kernel plus `kernels` (every product of the step timed
alone against its own roofline), and `cpu_baseline` (the CPU oracle, a restatement of the
reference's single-threaded CPU backend, timed on this host on a bounded sample).
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
    kind "softmax" / "adamw": the pointwise neighbours of the path (HBM-bound; reported in GB/s).
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
    "softmax": Workload("softmax", "row softmax fwd+bwd over the attention scores [8,12,512,512]",
                        (8, 12, 512, 512), (1, 1), kind="softmax"),
    "adamw": Workload("adamw", "gradient norm + clipped AdamW step on a [768,3072] weight and 64 M elements",
                      (64 * 1024 * 1024,), (1, 1), kind="adamw"),
}
HBM_BOUND = ("c3", "c5b1", "c5b4", "c5b16")
SHARDED = ("c4", "c5a")            # partition across ranks (strong scaling); c2 is weak-scaled; the rest are replicas
# DRAM bytes of one forward launch, from ncu captures of that launch summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum): a cited capture, not a measurement of this run.
NCU_TRAFFIC = {
    "c2": (34.11e6 + 19.63e6, "profiles/gemm_tc_kernel_c2_linear.md"),
    # captured on a 1/8 shard (34.7 MB read + 46.3 MB written of 135.3 MB algorithmic; the output's last ~54 MB stay
    # in L2) and scaled to 64 batches: operands 210.7 MB, output 805.3 MB minus the same L2 residue
    "c4": (210.7e6 + 805.3e6 - 54.4e6, "profiles/gemm_tc_kernel_c4_broadcast_weight.md (scaled from the 8-batch shard)"),
}
C5A_PANELS = 4                      # row panels of dB, each reduced as soon as it is computed


def shard_workload(wl: Workload, rank: int, world: int) -> Workload:
    """Per-rank shard for the configurations that partition: batch shards for c4, row shards for
    c5a.  c2 is weak-scaled (every rank owns a full-size batch shard), the rest run as replicas."""
    if world == 1 or wl.name not in SHARDED:
        return wl
    from framework_b200.sharding import shard_leading
    return wl.with_a_shape(shard_leading(wl.a_shape, rank, world), f" (1/{world} shard)")


def config_dict(base: Workload, world: int, precision: str) -> dict:
    """The `config` object: the same for this arm and for the reference arm."""
    if base.kind in ("softmax", "adamw"):
        par = "single GPU" if world == 1 else f"{world} replicas"
    elif world == 1:
        par = "single GPU"
    elif base.name == "c4":
        par = f"dp{world}: 64/{world} batches per rank, one NCCL reduce of dW (flat buffer) overlapped with the dA GEMM"
    elif base.name == "c5a":
        par = (f"dp{world}: 8192/{world} rows of A per rank, dB computed in {C5A_PANELS} row panels, each NCCL-reduced "
               "as it completes, overlapped with the next panel and the dA GEMM")
    elif base.name == "c2":
        par = f"dp{world}: one full-size batch shard per rank (weak), one NCCL reduce of dW+db (flat buffer)"
    else:
        par = f"{world} replicas (the configuration does not shard)"
    ws = working_set_mb(base)
    return {"workload": f"{base.name}: {base.desc}", "shapes": f"{base.a_shape} x {base.b_logical}",
            "parallelism": par, "precision": precision,
            "l2": (f"working set {ws:.0f} MB per step vs 126 MB L2, no flush" if ws > 126 else
                   f"working set {ws:.0f} MB fits the 126 MB L2; not flushed between steps (stated)"),
            "flops_per_step": None if base.kind in ("softmax", "adamw")
                              else (base.flops if base.name in SHARDED else base.flops * world)}


def scaling_label(base: Workload) -> str:
    return "strong" if base.name in SHARDED else "weak"


class Problem:
    """Device-side instance of a workload: resident inputs, preallocated outputs, the call sequence.

    The gradients that are summed over ranks (dW, db) are views of ONE flat buffer, so that a step
    needs one collective call for them."""

    def __init__(self, F, wl: Workload, host: dict, dev, flags: int, panels: int = 1):
        import torch
        T = F.DeviceTensor
        self.F, self.wl, self.flags = F, wl, flags
        self.inp = {k: T.from_numpy(v, dev) for k, v in host.items()}
        if wl.kind == "attention":
            self.kt = self.inp["k"].permute(wl.b_perm)
            shp = wl.out_shape
            self.out = {"s": T.empty(shp, dev), "o": T.empty(wl.a_shape, dev), "ds": T.empty(shp, dev),
                        "dv": T.empty(wl.a_shape, dev), "dq": T.empty(wl.a_shape, dev),
                        "dkt": T.empty(self.kt.shape, dev)}
            return
        self.b = self.inp["b"].permute(wl.b_perm) if wl.b_perm else self.inp["b"]
        n_w = int(np.prod(self.b.shape))
        n_b = wl.mkn[2] if wl.bias else 0
        off_b = (n_w + 63) // 64 * 64                       # 256-byte aligned start of db inside the flat buffer
        self.grad_flat = torch.empty(off_b + n_b if n_b else n_w, dtype=torch.float32, device=dev)
        self.out = {"y": T.empty(wl.out_shape, dev), "da": T.empty(wl.a_shape, dev),
                    "db": T(self.grad_flat[:n_w], self.b.shape)}
        if wl.bias:
            self.out["dbias"] = T(self.grad_flat[off_b:off_b + n_b], (n_b,))
        # Row panels of the weight gradient (2-D problems): rows [lo, hi) of dB = A[:, lo:hi]^T . dC need the
        # matching columns of A and land contiguously in the flat buffer.
        self.panels = []
        if panels > 1 and len(wl.a_shape) == 2 and not wl.bias:
            from framework_b200.sharding import panel_bounds
            k, n = self.b.shape
            for lo, hi in panel_bounds(k, panels, multiple=128):
                self.panels.append((self.inp["a"].narrow(1, lo, hi - lo), self.b.narrow(0, lo, hi - lo),
                                    T(self.grad_flat[lo * n:hi * n], (hi - lo, n)), self.grad_flat[lo * n:hi * n]))

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

    def backward_weight_panel(self, p: int):
        a_cols, b_rows, db_rows, _ = self.panels[p]
        self.F.matmul_backward(self.inp["dy"], a_cols, b_rows, flags=self.flags, need_da=False, db=db_rows)

    def backward_inputs(self):
        i, o = self.inp, self.out
        self.F.matmul_backward(i["dy"], i["a"], self.b, flags=self.flags, da=o["da"], need_db=False)

    def products(self):
        """Every GEMM of the step as (label, callable, algorithmic bytes, flops): each operand read once, the
        output written once."""
        F, i, o, fl = self.F, self.inp, self.out, self.flags
        wl = self.wl
        m, k, n = wl.mkn
        one = 2 * m * n * k * wl.batch

        def nbytes(*ts):
            return 4.0 * sum(int(np.prod(t.shape)) for t in ts)
        if wl.kind == "attention":
            return [
                ("S = Q.K^T", lambda: F.matmul(i["q"], self.kt, flags=fl, out=o["s"]), nbytes(i["q"], i["k"], o["s"]), one),
                ("O = S.V", lambda: F.matmul(o["s"], i["v"], flags=fl, out=o["o"]), nbytes(o["s"], i["v"], o["o"]), one),
                ("dS = dO.V^T", lambda: F.matmul_backward(i["do"], o["s"], i["v"], flags=fl, da=o["ds"], need_db=False),
                 nbytes(i["do"], i["v"], o["ds"]), one),
                ("dV = S^T.dO", lambda: F.matmul_backward(i["do"], o["s"], i["v"], flags=fl, need_da=False, db=o["dv"]),
                 nbytes(o["s"], i["do"], o["dv"]), one),
                ("dQ = dS.K", lambda: F.matmul_backward(o["ds"], i["q"], self.kt, flags=fl, da=o["dq"], need_db=False),
                 nbytes(o["ds"], i["k"], o["dq"]), one),
                ("dK^T = Q^T.dS", lambda: F.matmul_backward(o["ds"], i["q"], self.kt, flags=fl, need_da=False, db=o["dkt"]),
                 nbytes(i["q"], o["ds"], o["dkt"]), one),
            ]
        return [
            ("forward y = a.b" + (" + bias" if wl.bias else ""), self.forward, nbytes(i["a"], self.b, o["y"]), one),
            ("grad_a = dy.b^T", self.backward_inputs, nbytes(i["dy"], self.b, o["da"]), one),
            ("grad_b = a^T.dy" + (" (+ dbias)" if wl.bias else "") + (" (batch folded into K)" if wl.batch > 1 and len(wl.b_shape) == 2 else ""),
             self.backward_weights, nbytes(i["a"], i["dy"], o["db"]), one),
        ]


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


def load_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except OSError:
        return {}


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    import framework_b200 as F
    from framework_b200.sharding import DataParallelStep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    base = WORKLOADS[args.workload]
    nccl_ctas = args.nccl_ctas if args.nccl_ctas > 0 else (32 if (base.name == "c5a" and world >= 8) else 16)
    if args.sm_reserve < 0:
        args.sm_reserve = 2 if world >= 8 else 1
    if world > 1:
        # The reduce runs beside persistent one-CTA-per-SM grids: cap the SMs it may take, and leave as many free.
        os.environ.setdefault("NCCL_MAX_CTAS", str(nccl_ctas))
        dist.init_process_group("nccl", device_id=dev)

    if base.kind in ("softmax", "adamw"):
        run_pointwise(args, F, base, dev, world, rank)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    wl = shard_workload(base, rank, world)
    if world == 1 and args.shard_of > 1:     # one rank's shard of an N-rank run, alone on this GPU (no reduce): kernel tuning
        wl = shard_workload(base, 0, args.shard_of)
    flags = F._lib.PRECISION_TF32 if args.precision == "tf32" else 0
    host = wl.host_inputs(seed=rank)
    if world > 1 and wl.kind == "gemm":      # the weight (and bias) are replicated
        shared = wl.host_inputs(seed=0)
        for key in ("b", "bias"):
            if key in host:
                host[key] = shared[key]
    reduce_grads = world > 1 and wl.name in ("c2", "c4", "c5a")
    n_panels = C5A_PANELS if (reduce_grads and wl.name == "c5a") else 1
    prob = Problem(F, wl, host, dev, flags, panels=n_panels)

    # Data parallel: the weight gradient is computed first (for c5a in row panels) and summed onto rank 0 on a
    # second stream while the next panel, the input-gradient GEMM and the next step's forward run.
    comm = torch.cuda.Stream() if reduce_grads else None

    def make_step(pr):
        if wl.kind == "attention":
            def plain():
                pr.forward()
                pr.backward()
            plain.join = lambda: None
            return plain
        if not reduce_grads:
            def plain():
                pr.forward()
                pr.backward()
            plain.join = lambda: None
            return plain
        if pr.panels:
            fns = [(lambda p=p: pr.backward_weight_panel(p)) for p in range(len(pr.panels))]
            bufs = [p[3] for p in pr.panels]
        else:
            fns, bufs = [pr.backward_weights], [pr.grad_flat]
        return DataParallelStep(pr.forward, fns, bufs, pr.backward_inputs, streams=(torch.cuda.current_stream(), comm),
                                everywhere=args.collective == "allreduce",
                                reserve=F.sm_reserve if args.sm_reserve else None, reserve_sms=nccl_ctas,
                                reserve_forward=args.sm_reserve >= 2)

    eager_step = make_step(prob)

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
    eager_step.join()
    F.device_status()

    # Launch-bound workloads replay the step from a CUDA graph (same kernels, same order).
    step, graphed = eager_step, False
    est_ms = timed(eager_step, 5, after=eager_step.join) / 5
    eager_ms = est_ms
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
        eager_ms = timed(eager_step, 50) / 50

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    launches0 = F.launch_count()
    eager_step()
    launches_per_step = F.launch_count() - launches0
    eager_step.join()
    torch.cuda.synchronize()
    t_wall0 = time.time()
    total_ms = timed(step, args.steps, after=eager_step.join)
    t_wall1 = time.time()
    F.device_status()
    ms_per_step = total_ms / args.steps
    value = wl.flops * world / (ms_per_step * 1e-3) / 1e12
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None

    # ---- phase timeline of one step on rank 0 (multi-GPU only): where the reduce sits beside the GEMMs -----
    timeline = None
    if reduce_grads:
        marks = []

        def mark(label, stream):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            marks.append((label, ev))
        for _ in range(2):
            marks.clear()
            barrier()
            eager_step(mark)
            eager_step.join()
            barrier()
        if rank == 0:
            t0 = marks[0][1]
            timeline = {label: round(t0.elapsed_time(ev) * 1e3, 1) for label, ev in marks}
            timeline["unit"] = "us after step begin, rank 0, one eager step between barriers"

    # ---- rooflines: every product of the step timed alone (burst clocks: let the power state settle first) ----
    peaks = load_peaks()
    torch.cuda.synchronize()
    time.sleep(0.5)
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    tf32_peak = peaks.get("bf16_tflops", 1590.0) / 2.0
    hbm_bound = wl.name in HBM_BOUND
    kernels = []
    reps = max(5, min(args.steps, 50))
    # Launch-bound workloads: each product is replayed from its own CUDA graph, like the step.  The skinny
    # products stream one 67 MB weight that would otherwise stay in the 126 MB L2 from call to call: three
    # problem instances (three weights) take turns, so every call finds its weight in HBM.
    rotation = [prob]
    if graphed and wl.name.startswith("c5b"):
        rotation += [Problem(F, wl, wl.host_inputs(seed=100 + i), dev, flags) for i in range(2)]
    product_lists = [pr.products() for pr in rotation]
    for idx, (label, fn, alg_bytes, flops) in enumerate(product_lists[0]):
        fns = [pl[idx][1] for pl in product_lists]

        def run_all(fns=fns):
            for f in fns:
                f()
        l0 = F.launch_count()
        fn()
        n_launch = F.launch_count() - l0
        how = "eager calls back to back"
        if graphed:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run_all()
            torch.cuda.current_stream().wait_stream(side)
            gp = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gp):
                run_all()
            for _ in range(3):
                gp.replay()
            ms = timed(gp.replay, reps) / reps / len(fns)
            how = "CUDA-graph replay" + (f", {len(fns)} weights in turn (none stays in L2)" if len(fns) > 1 else "")
        else:
            ms = timed(run_all, reps) / reps / len(fns)
        gbs = alg_bytes / (ms * 1e-3) / 1e9
        tfs = flops / (ms * 1e-3) / 1e12
        entry = {"call": label, "us": round(ms * 1e3, 2), "launches": n_launch, "tflops": round(tfs, 2),
                 "gbs": round(gbs, 1), "algorithmic_bytes": alg_bytes, "timed": how}
        if hbm_bound:
            entry.update(bound="hbm", frac=round(gbs / hbm_peak, 4))
        else:
            issued = tfs * (1 if args.precision == "tf32" else 3)
            entry.update(bound="tensor", frac=round(tfs / tf32_peak, 4), issued_frac=round(issued / tf32_peak, 4))
        kernels.append(entry)
    first = kernels[0]
    if hbm_bound:
        total_bytes = sum(k["algorithmic_bytes"] for k in kernels)
        total_us = sum(k["us"] for k in kernels)
        roofline = {"bound": "hbm", "achieved": first["gbs"], "peak": hbm_peak, "unit": "GB/s",
                    "frac": first["gbs"] / hbm_peak, "traffic": None,
                    "kernel": f"{first['call']} ({first['launches']} launch(es); the other products are in `kernels`)",
                    "algorithmic_bytes": first["algorithmic_bytes"],
                    "all_products": {"gbs": round(total_bytes / (total_us * 1e-6) / 1e9, 1),
                                     "frac": round(total_bytes / (total_us * 1e-6) / 1e9 / hbm_peak, 4),
                                     "note": "sum of algorithmic bytes / sum of the products' stand-alone times"},
                    "peak_source": "measured hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650"}
    else:
        traffic, source = (NCU_TRAFFIC.get(wl.name, (None, None))
                           if (args.precision != "tf32" and world == 1 and args.shard_of == 1) else (None, None))
        issued = first["tflops"] * (1 if args.precision == "tf32" else 3)
        roofline = {"bound": "tensor", "achieved": first["tflops"], "peak": tf32_peak, "unit": "TFLOP/s",
                    "frac": first["tflops"] / tf32_peak, "traffic": traffic,
                    "traffic_source": (f"cited from {source} (ncu dram read+write bytes of this launch), not measured by this run"
                                       if source else None),
                    "algorithmic_bytes": first["algorithmic_bytes"],
                    "kernel": f"gemm_tc_kernel ({first['call']}; the other products are in `kernels`)",
                    "issued_tflops": issued, "issued_frac": issued / tf32_peak,
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
    slots = [prob, Problem(F, wl, host, dev, flags, panels=n_panels)]
    slot_steps = [eager_step, make_step(slots[1])]
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
        slot_steps[i]()
        slot_steps[i].join()
        ev_done[i].record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[i])
            for key, h in h_out.items():
                t = pr.out[key]
                h.copy_(t.storage[: t.size], non_blocking=True)
            ev_out[i].record(s_out)

    def e2e_join():
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

    # Last measurement of the run (it heats the GPU to its power cap).  NVML refreshes its clock and throttle
    # readings far more slowly than a timed region of ~0.1 s lasts, so the same steps are repeated, untimed, for
    # about a second with a second sampler: what the clocks settle at under this workload, reported beside the
    # readings taken during the timed region.
    sustain_steps = int(min(20000, max(args.steps, 1000.0 / max(ms_per_step, 1e-3))))
    sustain = ClockSampler(local_rank)
    if rank == 0:
        sustain.start()
    t_s0 = time.time()
    sustain_ms = timed(step, sustain_steps, after=eager_step.join)
    t_s1 = time.time()
    if rank == 0:
        settled = sustain.stop(t_s0 + 0.5 * (t_s1 - t_s0), t_s1)       # second half of the window
        clocks["sustained"] = {"seconds": round(t_s1 - t_s0, 2), "steps": sustain_steps,
                               "ms_per_step": sustain_ms / sustain_steps,
                               "value": wl.flops * world / (sustain_ms / sustain_steps * 1e-3) / 1e12,
                               "sm_mhz": settled.get("sm_mhz"),
                               "sm_min_mhz": settled.get("sm_min_mhz"), "power_w_max": settled.get("power_w_max"),
                               "reasons": settled.get("reasons"), "samples": settled.get("samples")}
        for r in settled.get("reasons") or []:
            if r not in clocks["reasons"]:
                clocks["reasons"].append(r)

    if rank == 0:
        cpu = cpu_baseline_sample(base, threads=1) if (world == 1 and not args.no_cpu) else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": scaling_label(base), "vs_baseline": None,
            "dtype": "f32 storage, 3xTF32 tensor-core arithmetic (f32 accumulate)" if args.precision != "tf32"
                     else "f32 storage, single-pass TF32 arithmetic (reduced precision mode)",
            "data": "synthetic (seeded numpy default_rng: x~U[0,1), W~N(0,0.02), b~N(0,0.02), dy~N(0,1))"
                    if wl.name == "c2" else "synthetic (seeded numpy default_rng, ~N(0,1); weight ~N(0,0.02))"
                    if wl.name == "c4" else "synthetic (seeded numpy default_rng, ~N(0,1))",
            "config": config_dict(base, world, args.precision),
            "run": {"per_gpu": f"{wl.a_shape} x {wl.b_logical}", "cuda_graph": graphed, "shard_of": args.shard_of,
                    "nccl_max_ctas": nccl_ctas if world > 1 else None, "sm_reserve": args.sm_reserve if world > 1 else None,
                    "collective": args.collective if world > 1 else None,
                    "eager_ms_per_step": eager_ms, "flops_per_step_per_gpu": wl.flops},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "overlap": "3 streams, 2 device slots"},
            "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks,
            "roofline": roofline,
            "kernels": kernels,
        }
        if timeline is not None:
            line["timeline"] = timeline
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_pointwise(args, F, base: Workload, dev, world: int, rank: int):
    """The HBM-bound neighbours of the path: softmax forward+backward over the attention scores, and the
    gradient-norm + clipped AdamW step that consumes dW.  Reported in GB/s of algorithmic bytes."""
    import torch
    T = F.DeviceTensor
    rng = np.random.default_rng(rank)
    peaks = load_peaks()
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    if base.kind == "softmax":
        shape = base.a_shape
        x = T.from_numpy(rng.standard_normal(shape, dtype=np.float32), dev)
        dy = T.from_numpy(rng.standard_normal(shape, dtype=np.float32), dev)
        y = F.softmax(x, -1)
        n = int(np.prod(shape))
        parts = [("softmax forward", lambda: F.softmax(x, -1), 8.0 * n),
                 ("softmax backward", lambda: F.softmax_backward(dy, y, -1), 12.0 * n)]
        host_in = {"x": x, "dy": dy}
        outs = lambda: {"y": F.softmax(x, -1), "dx": F.softmax_backward(dy, F.softmax(x, -1), -1)}  # noqa: E731
    else:
        sizes = [768 * 3072, base.a_shape[0]]
        ps = [T.from_numpy(rng.standard_normal(s, dtype=np.float32), dev) for s in sizes]
        gs = [T.from_numpy(rng.standard_normal(s, dtype=np.float32), dev) for s in sizes]
        ms = [T.from_numpy(np.zeros(s, np.float32), dev) for s in sizes]
        vs = [T.from_numpy(np.zeros(s, np.float32), dev) for s in sizes]
        sumsq = torch.zeros(1, dtype=torch.float64, device=dev)
        lib = F._lib.lib()
        from framework_b200.tensor import current_stream

        def norm():
            for i, g in enumerate(gs):
                F._lib.check(lib.mni_b200_grad_sumsq(g.ptr, g.size, sumsq.data_ptr(), F._lib.ACCUMULATE_C if i else 0,
                                                     current_stream()))

        def step_all():
            for p, m, v, g in zip(ps, ms, vs, gs):
                F.adamw_step(p, m, v, g, lr=1e-3, weight_decay=0.01, step=3, grad_sumsq=sumsq, max_grad_norm=1.0,
                             write_clipped_grad=False)
        n = sum(sizes)
        parts = [("gradient norm (f64 sum of squares)", norm, 4.0 * n),
                 ("clipped AdamW step (param, m, v read+written, grad read)", step_all, 28.0 * n)]
        host_in, outs = {}, None
    kernels, total_ms, total_bytes = [], 0.0, 0.0
    reps = max(5, min(args.steps, 100))
    for label, fn, nbytes in parts:
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = F.launch_count()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms_ = e0.elapsed_time(e1) / reps
        gbs = nbytes / (ms_ * 1e-3) / 1e9
        kernels.append({"call": label, "us": round(ms_ * 1e3, 2), "launches": (F.launch_count() - l0) // reps,
                        "gbs": round(gbs, 1), "algorithmic_bytes": nbytes, "bound": "hbm", "frac": round(gbs / hbm_peak, 4)})
        total_ms += ms_
        total_bytes += nbytes
    F.device_status()
    if rank != 0:
        return
    value = total_bytes / (total_ms * 1e-3) / 1e9
    line = {"metric": f"{base.name}_algorithmic_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": reps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded numpy default_rng, ~N(0,1))",
            "config": config_dict(base, world, "f32"),
            "roofline": {"bound": "hbm", "achieved": value, "peak": hbm_peak, "unit": "GB/s", "frac": value / hbm_peak,
                         "traffic": None, "kernel": "all calls of the workload, back to back",
                         "peak_source": "measured hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650"},
            "kernels": kernels, "gpu_launches": int(sum(k["launches"] for k in kernels) * reps)}
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline_pointwise(base)
    print(json.dumps(line), flush=True)


def working_set_mb(wl: Workload) -> float:
    if wl.kind == "attention":
        elems = 2 * np.prod(wl.out_shape) + 8 * np.prod(wl.a_shape)
    elif wl.kind in ("softmax", "adamw"):
        elems = 4 * np.prod(wl.a_shape)
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


def cpu_rate_gflops(O, threads: int) -> float:
    """Quick calibration of the CPU loop's speed (a 512 x 512 x 2048 product per thread) so that samples can be
    sized in seconds rather than in flops."""
    m = 512 * max(threads, 1)
    rng = np.random.default_rng(1)
    a = O.HostTensor.from_array(rng.standard_normal((m, 512), dtype=np.float32))
    b = O.HostTensor.from_array(rng.standard_normal((512, 2048), dtype=np.float32))
    O.matmul(a, b, threads=threads)
    t0 = time.perf_counter()
    O.matmul(a, b, threads=threads)
    return 2.0 * m * 512 * 2048 / (time.perf_counter() - t0) / 1e9


def cpu_baseline_sample(wl: Workload, threads: int) -> dict:
    import oracle as O
    O.build()
    rate = cpu_rate_gflops(O, threads)
    small, what = cpu_sample_workload(wl, budget_gflop=max(1.0, 12.0 * rate))     # about 12 s of CPU work
    tens = cpu_tensors(O, small)
    t0 = time.perf_counter()
    cpu_step(O, small, tens, threads)
    dt = time.perf_counter() - t0
    return {"value": small.flops / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{what}; {small.flops / 1e9:.1f} GFLOP in {dt:.2f} s; C restatement of the reference's "
                      f"single-threaded CPU backend (gcc -O3 -ffp-contract=off)",
            "host_cores": host_threads()}


def cpu_baseline_pointwise(base: Workload) -> dict:
    import oracle as O
    O.build()
    rng = np.random.default_rng(0)
    if base.kind == "softmax":
        shape = (2,) + tuple(base.a_shape[1:])                       # 2 of the 8 batches
        x = rng.standard_normal(shape, dtype=np.float32)
        dy = rng.standard_normal(shape, dtype=np.float32)
        t0 = time.perf_counter()
        y = O.softmax(x, -1)
        O.softmax_backward(dy, y, -1)
        dt = time.perf_counter() - t0
        nbytes, what = 20.0 * x.size, "2/8 of the batches, forward + backward"
    else:
        n = 16 * 1024 * 1024
        p, g = rng.standard_normal(n, dtype=np.float32), rng.standard_normal(n, dtype=np.float32)
        m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
        t0 = time.perf_counter()
        O.clip_and_step([p], [m], [v], [g], lr=1e-3, weight_decay=0.01, step=3, max_grad_norm=1.0)
        dt = time.perf_counter() - t0
        nbytes, what = 32.0 * n, "16 M elements, norm + clip + AdamW"
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": f"{what}; {dt:.2f} s; C restatement of the reference's single-threaded CPU backend",
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
    if wl.kind in ("softmax", "adamw"):
        cpu = cpu_baseline_pointwise(wl)
        print(json.dumps({"impl": "reference", "metric": f"{wl.name}_algorithmic_gbs", "value": cpu["value"], "unit": "GB/s",
                          "n_gpus": world, "steps": 1, "warmup": 0, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(wl, world, "f32"),
                          "cpu_baseline": cpu, "e2e": {"value": cpu["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                                                       "d2h_bytes_per_step": 0}}), flush=True)
        return
    # Size the per-step sample so that all warm-up and timed steps together take about 90 s of CPU time.
    steps, warm = max(1, args.steps), max(0, args.warmup)
    rate = cpu_rate_gflops(O, threads)
    small, what = cpu_sample_workload(wl, budget_gflop=max(0.5, 90.0 / (steps + warm) * rate))
    tens = cpu_tensors(O, small)
    for _ in range(warm):
        cpu_step(O, small, tens, threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(O, small, tens, threads)
    dt = (time.perf_counter() - t0) / steps
    value = small.flops / dt / 1e12
    sample = (f"{what}; {small.flops / 1e9:.1f} GFLOP per step, {steps} timed steps; the reference's CPU backend is "
              f"single-threaded, this run spreads its row loop over {threads} threads (bit-identical results)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": scaling_label(wl),
        "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded numpy default_rng)",
        "config": config_dict(wl, world, args.precision),
        "run": {"threads": threads, "calibrated_gflops": round(rate, 1)},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--precision", default="3xtf32", choices=["3xtf32", "tf32"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the step from a CUDA graph (auto: only for steps under 0.2 ms)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--nccl-ctas", type=int, default=0,
                    help="cap on the SMs the NCCL reduce may use (NCCL_MAX_CTAS); default 16 (32 for c5a's 268 MB at 8 ranks: measured 1883 vs 1775 TFLOP/s there, but 936 vs 1001 at 4 ranks and 463 vs 502 at 2)")
    ap.add_argument("--sm-reserve", type=int, default=-1,
                    help="1: the GEMMs that run beside the reduce leave that many SMs free; 2: the next forward too; "
                         "0: they use every SM; default: 2 from 8 ranks on (the reduce outlasts the input-gradient "
                         "GEMM there), else 1")
    ap.add_argument("--collective", default="reduce", choices=["reduce", "allreduce"],
                    help="sum of the weight gradient: onto rank 0 (ncclReduce) or onto every rank (ncclAllReduce)")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="with one GPU: run rank 0's shard of an N-rank job (c4 / c5a), without the reduce")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
