"""Sharding of the matmul path over the GPUs of one node.

The forward and the input gradient partition with no exchange: batches (broadcast-weight
GEMM) or rows of A (plain 2-D GEMM) are independent.  Only the gradient of the operand
every shard shares -- the weight, and the bias -- needs one sum over ranks, onto rank 0.
One process per GPU; `torch.distributed` carries the reduce (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

from typing import Sequence, Tuple


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


def reduce_to_root(flat, dst: int = 0, group=None) -> None:
    """Sums a flat gradient buffer over all ranks onto `dst` (in place on dst)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.reduce(flat, dst=dst, op=dist.ReduceOp.SUM, group=group)
