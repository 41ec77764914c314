"""Device tensor with the reference's data model: storage + shape + element strides.

Mirrors ``GpuTensor`` of src/native/src/tensor.rs:63-73.  ``permute`` is a
stride-only view (what the reference's CPU backend does, ops/layout.rs:112-134;
its CUDA backend materialises instead, :137-156) so that strided operands reach
the matmul kernels through TMA descriptors without a copy.  PyTorch is used only
to own device memory and to name the current stream.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from . import _lib


def row_major_strides(shape: Sequence[int]) -> tuple:
    """tensor.rs:7-17 compute_strides."""
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= int(s)
    return tuple(reversed(st))


def shape_size(shape: Sequence[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def current_stream() -> int:
    return int(torch.cuda.current_stream().cuda_stream)


class DeviceTensor:
    """f32 tensor on the current CUDA device: flat storage, shape, element strides."""

    __slots__ = ("storage", "shape", "strides")

    def __init__(self, storage: torch.Tensor, shape: Sequence[int], strides: Sequence[int] | None = None):
        if storage.dtype != torch.float32 or not storage.is_cuda or storage.dim() != 1:
            raise TypeError("storage must be a flat float32 CUDA tensor")
        self.storage = storage
        self.shape = tuple(int(s) for s in shape)
        self.strides = tuple(int(s) for s in strides) if strides is not None else row_major_strides(self.shape)

    # -- construction ------------------------------------------------------
    @staticmethod
    def empty(shape: Sequence[int], device=None) -> "DeviceTensor":
        n = max(shape_size(shape), 1)
        return DeviceTensor(torch.empty(n, dtype=torch.float32, device=device or "cuda"), shape)

    @staticmethod
    def from_numpy(a: np.ndarray, device=None) -> "DeviceTensor":
        """Tensor.fromFloat32 (src/tensor.ts:72-75): host f32 data -> contiguous device tensor."""
        a = np.ascontiguousarray(a, dtype=np.float32)
        flat = torch.from_numpy(a.reshape(-1))
        return DeviceTensor(flat.to(device or "cuda"), a.shape)

    @staticmethod
    def from_torch(t: torch.Tensor) -> "DeviceTensor":
        """Wraps a CUDA f32 torch tensor (any strides) without copying."""
        if t.dtype != torch.float32 or not t.is_cuda:
            raise TypeError("need a float32 CUDA tensor")
        base = t.untyped_storage()
        flat = torch.empty(0, dtype=torch.float32, device=t.device).set_(
            base, t.storage_offset(), (max(_span(t), 1),), (1,))
        return DeviceTensor(flat, tuple(t.shape), tuple(t.stride()))

    # -- properties --------------------------------------------------------
    @property
    def size(self) -> int:
        return shape_size(self.shape)

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def ptr(self) -> int:
        return int(self.storage.data_ptr())

    def is_contiguous(self) -> bool:
        """tensor.rs:77-89."""
        return self.strides == row_major_strides(self.shape)

    def view_struct(self) -> "_lib.View":
        return _lib.make_view(self.ptr, self.shape, self.strides)

    # -- layout ops (ops/layout.rs) ------------------------------------------
    def permute(self, dims: Sequence[int]) -> "DeviceTensor":
        """Stride-only permutation sharing the storage (no kernel, no copy)."""
        if sorted(dims) != list(range(self.ndim)):
            raise ValueError(f"invalid permutation {list(dims)}")
        return DeviceTensor(self.storage, [self.shape[d] for d in dims], [self.strides[d] for d in dims])

    def narrow(self, dim: int, start: int, length: int) -> "DeviceTensor":
        """The sub-tensor [start, start + length) of dimension `dim`, as a view of the same storage (pointer
        offset + same strides): how row or column panels of an operand reach the kernels without a copy."""
        d = dim + self.ndim if dim < 0 else dim
        if not (0 <= d < self.ndim and 0 <= start and length >= 0 and start + length <= self.shape[d]):
            raise ValueError(f"narrow({dim}, {start}, {length}) out of range for shape {self.shape}")
        shape = list(self.shape)
        shape[d] = length
        return DeviceTensor(self.storage[start * self.strides[d]:], shape, self.strides)

    def contiguous(self) -> "DeviceTensor":
        """ops/layout.rs:218-231 / tensor.rs:510-517, done on the device."""
        if self.is_contiguous():
            return self
        out = DeviceTensor.empty(self.shape, self.storage.device)
        v = self.view_struct()
        _lib.check(_lib.lib().mni_b200_contiguous(v, out.ptr, current_stream()))
        return out

    def view(self, shape: Sequence[int]) -> "DeviceTensor":
        """ops/layout.rs:80-89: reshape of the contiguous data (shares storage when already contiguous)."""
        if shape_size(shape) != self.size:
            raise ValueError(f"cannot view {self.shape} as {tuple(shape)}")
        return DeviceTensor(self.contiguous().storage, shape)

    # -- host transfer -----------------------------------------------------
    def numpy(self) -> np.ndarray:
        """toFloat32 (tensor.rs:364-387): logical contents, row-major."""
        c = self.contiguous()
        return c.storage[: max(c.size, 0)].cpu().numpy().reshape(c.shape).copy()

    def torch_view(self) -> torch.Tensor:
        """The same memory as a strided torch tensor (for harness comparisons)."""
        return torch.as_strided(self.storage, self.shape, self.strides)


def _span(t: torch.Tensor) -> int:
    if t.numel() == 0:
        return 0
    return 1 + sum((s - 1) * st for s, st in zip(t.shape, t.stride()))
