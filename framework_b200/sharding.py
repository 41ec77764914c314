"""Sharding of the matmul path over the GPUs of one node.

The forward and the input gradient partition with no exchange: batches (broadcast-weight
GEMM) or rows of A (plain 2-D GEMM) are independent.  Only the gradient of the operand
every shard shares -- the weight, and the bias -- needs one sum over ranks, onto rank 0:
the device-side replacement of the host-side reduction the reference runs for a broadcast
weight gradient (ops/matmul.rs:243-251, utils.rs:39-66).
One process per GPU; `torch.distributed` carries the reduce (NCCL on GPUs, gloo in CPU tests).

`DataParallelStep` is the step driver both use: weight gradient first, its reduce on a second
stream, input gradient (and the next forward) beside it.  It only sees callables and flat
buffers, so the CPU tests run the same function with the oracle standing in for the kernels.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open range of the `n` leading units owned by `rank`; the first n % world ranks get one more."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, rem = divmod(int(n), world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_leading(shape: Sequence[int], rank: int, world: int) -> tuple:
    """Shape of rank's shard when the leading dim (batch, or rows of a 2-D A) is split."""
    lo, hi = shard_bounds(shape[0], rank, world)
    return (hi - lo,) + tuple(shape[1:])


def panel_bounds(n: int, panels: int, multiple: int = 1) -> List[Tuple[int, int]]:
    """Cuts range(n) into at most `panels` contiguous pieces whose boundaries are multiples of `multiple`."""
    panels = max(1, min(int(panels), max(1, n // max(multiple, 1))))
    edges = [min(n, ((n * i // panels) + multiple - 1) // multiple * multiple) for i in range(panels)] + [n]
    return [(lo, hi) for lo, hi in zip(edges[:-1], edges[1:]) if hi > lo]


def reduce_to_root(flat, dst: int = 0, group=None, everywhere: bool = False) -> None:
    """Sums a flat gradient buffer over all ranks onto `dst` (in place on dst).  With `everywhere` the sum is
    left on every rank (an all-reduce): what replicas that each apply the optimizer step need, and on NVSwitch
    systems the form NCCL can reduce inside the switch."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        if everywhere:
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        else:
            dist.reduce(flat, dst=dst, op=dist.ReduceOp.SUM, group=group)


class DataParallelStep:
    """One forward+backward step of a shard whose weight gradient is summed onto rank 0.

    forward()                  the shard's forward
    weight_grad_panels         callables, each computing one panel of the weight gradient (and, in the
                               first, the bias gradient) into its slice of ONE flat buffer
    panel_buffers              the flat tensors those panels fill, in the same order; each is reduced
                               as soon as its panel is done -- one collective call per panel, on the
                               communication stream, while the next panel / the input gradient computes
    input_grad()               the shard's input gradient (no exchange)

    With `streams` = (main, comm) CUDA streams the reduce overlaps the compute; with None (CPU tests)
    everything runs in order.  `reserve(n)` (optional; `framework_b200.sm_reserve`) is called with
    `reserve_sms` before the first launch that runs beside a reduce and with 0 after the last: the
    tensor-core grids are persistent, one CTA per SM, so the collective's CTAs need SMs of their own or
    they push as many CTAs of the grid into a late second wave.
    """

    def __init__(self, forward: Callable[[], None], weight_grad_panels: Sequence[Callable[[], None]],
                 panel_buffers: Sequence, input_grad: Callable[[], None], *, streams=None, dst: int = 0,
                 group=None, reduce: bool = True, everywhere: bool = False,
                 reserve: Optional[Callable[[int], None]] = None, reserve_sms: int = 0, reserve_forward: bool = False):
        if len(weight_grad_panels) != len(panel_buffers):
            raise ValueError("one flat buffer per weight-gradient panel")
        self.forward, self.panels, self.buffers, self.input_grad = forward, list(weight_grad_panels), list(panel_buffers), input_grad
        self.streams, self.dst, self.group, self.reduce = streams, dst, group, reduce
        self.reserve = reserve if (reserve is not None and reserve_sms > 0 and reduce) else None
        self.reserve_sms = reserve_sms
        self.reserve_forward = reserve_forward      # the reduce may outlast the input gradient: keep the SMs free through the next forward
        self.everywhere = everywhere
        self._ev_panel: list = []
        self._ev_reduced = None
        if streams is not None:
            import torch
            self._ev_panel = [torch.cuda.Event() for _ in self.panels]
            self._ev_reduced = torch.cuda.Event()

    def __call__(self, mark: Optional[Callable[[str, object], None]] = None) -> None:
        if self.streams is None:
            self.forward()
            for fn, buf in zip(self.panels, self.buffers):
                fn()
                if self.reduce:
                    reduce_to_root(buf, self.dst, self.group, self.everywhere)
            self.input_grad()
            return
        import torch
        main, comm = self.streams
        if mark:
            mark("step begin", main)
        self.forward()
        if mark:
            mark("forward done", main)
        if self.reduce:
            main.wait_event(self._ev_reduced)        # the previous step's reduce is done with the gradient buffers
        if self.reserve:
            self.reserve(0)                          # nothing runs beside the first weight-gradient panel
        for i, (fn, buf) in enumerate(zip(self.panels, self.buffers)):
            fn()
            if mark:
                mark(f"weight grad panel {i} done", main)
            if not self.reduce:
                continue
            self._ev_panel[i].record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(self._ev_panel[i])
                if mark:
                    mark(f"reduce {i} begin", comm)
                reduce_to_root(buf, self.dst, self.group, self.everywhere)
                if mark:
                    mark(f"reduce {i} end", comm)
            if self.reserve:
                self.reserve(self.reserve_sms)     # everything launched from here on runs beside a reduce
        if self.reduce:
            self._ev_reduced.record(comm)
        self.input_grad()
        if self.reserve and not self.reserve_forward:
            self.reserve(0)
        if mark:
            mark("input grad done", main)

    def join(self) -> None:
        """Makes the main stream wait for the last reduce (end of a timed region, or before reading dW)."""
        if self.reserve:
            self.reserve(0)
        if self.streams is not None and self.reduce:
            self.streams[0].wait_event(self._ev_reduced)
