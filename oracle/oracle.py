"""ctypes front end of the C oracle (``mni_oracle.c``) -- test infrastructure only.

``HostTensor`` mirrors the reference's CPU ``GpuTensor`` (tensor.rs:27-37): a flat
f32 buffer plus ``shape`` and element ``strides``; ``permute`` is the stride-only
view of ops/layout.rs:112-134.  The arithmetic lives in C so that the multiply
and the add of each term stay separate f32 operations.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from typing import Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmni_oracle.so")
_lib = None

_i64p = C.POINTER(C.c_int64)
_f32p = C.POINTER(C.c_float)


def build(force: bool = False) -> str:
    """Compile ``libmni_oracle.so`` with the recipe in ``oracle/Makefile``."""
    src = os.path.join(_HERE, "mni_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "libmni_oracle.so"])
    return _SO


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.oracle_matmul_fwd.restype = C.c_int
        _lib.oracle_matmul_bwd.restype = C.c_int
        _lib.oracle_add.restype = C.c_int
        _lib.oracle_max_threads.restype = C.c_int
    return _lib


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def _shape_size(shape: Sequence[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return max(n, 1)


def _row_major(shape: Sequence[int]) -> tuple:
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= int(s)
    return tuple(reversed(st))


def _i64(v: Sequence[int]):
    return (C.c_int64 * max(len(v), 1))(*[int(x) for x in v])


def _fp(a: np.ndarray):
    return a.ctypes.data_as(_f32p)


@dataclass
class HostTensor:
    """Flat f32 storage + shape + element strides (tensor.rs:27-37)."""
    data: np.ndarray
    shape: tuple
    strides: tuple

    @staticmethod
    def from_array(a: np.ndarray) -> "HostTensor":
        a = np.ascontiguousarray(a, dtype=np.float32)
        return HostTensor(a.reshape(-1).copy(), tuple(a.shape), _row_major(a.shape))

    def is_contiguous(self) -> bool:  # tensor.rs:41-53
        return tuple(self.strides) == _row_major(self.shape)

    def numpy(self) -> np.ndarray:
        """Logical contents as an ndarray (gathers a strided view)."""
        return contiguous(self).data.reshape(self.shape)


def contiguous(t: HostTensor) -> HostTensor:
    """tensor.rs:311-318 ensure_contiguous."""
    if t.is_contiguous():
        return t
    out = np.empty(_shape_size(t.shape), np.float32)
    lib().oracle_make_contiguous(_fp(t.data), _i64(t.shape), _i64(t.strides),
                                 C.c_int(len(t.shape)), _fp(out))
    return HostTensor(out, tuple(t.shape), _row_major(t.shape))


def permute(t: HostTensor, dims: Sequence[int]) -> HostTensor:
    """ops/layout.rs:112-134: stride-only view over a clone of the storage."""
    return HostTensor(t.data.copy(), tuple(t.shape[d] for d in dims),
                      tuple(t.strides[d] for d in dims))


def permute_backward(grad: HostTensor, dims: Sequence[int], orig_shape: Sequence[int]) -> HostTensor:
    """ops/layout.rs:162-195."""
    g = contiguous(grad)
    out = np.empty(_shape_size(orig_shape), np.float32)
    lib().oracle_permute_bwd(_fp(g.data), _i64(g.shape), C.c_int(len(dims)), _i64(dims),
                             _i64(orig_shape), _fp(out))
    return HostTensor(out, tuple(orig_shape), _row_major(orig_shape))


def _bshape(a: Sequence[int], b: Sequence[int]) -> tuple:
    out = (C.c_int64 * 8)()
    nd = lib().oracle_broadcast_shape(_i64(a), C.c_int(len(a)), _i64(b), C.c_int(len(b)), out)
    if nd < 0:
        raise ValueError(f"shapes {list(a)} and {list(b)} are not broadcastable")
    return tuple(out[i] for i in range(nd))


_ERR = {-1: "matmul requires at least 2D tensors",
        -2: "matmul inner dimensions must match",
        -3: "shapes are not broadcastable", -4: "out of memory"}


def matmul(a: HostTensor, b: HostTensor, threads: int = 0) -> HostTensor:
    """ops/matmul.rs:19-78 (CPU backend forward)."""
    if len(a.shape) < 2 or len(b.shape) < 2:
        raise ValueError(_ERR[-1])
    if a.shape[-1] != b.shape[-2]:
        raise ValueError(f"{_ERR[-2]}: {a.shape[-1]} vs {b.shape[-2]}")
    oshape = _bshape(a.shape[:-2], b.shape[:-2]) + (a.shape[-2], b.shape[-1])
    out = np.empty(_shape_size(oshape), np.float32)
    rc = lib().oracle_matmul_fwd(_fp(a.data), _i64(a.shape), _i64(a.strides), C.c_int(len(a.shape)),
                                 _fp(b.data), _i64(b.shape), _i64(b.strides), C.c_int(len(b.shape)),
                                 _fp(out), C.c_int(threads or max_threads()))
    if rc:
        raise ValueError(_ERR.get(rc, str(rc)))
    return HostTensor(out, oshape, _row_major(oshape))


def matmul_backward(grad: HostTensor, a: HostTensor, b: HostTensor, threads: int = 0):
    """ops/matmul.rs:200-222 (CPU backend backward) -> (grad_a, grad_b)."""
    g = contiguous(grad)
    da = np.empty(_shape_size(a.shape), np.float32)
    db = np.empty(_shape_size(b.shape), np.float32)
    rc = lib().oracle_matmul_bwd(_fp(g.data), _i64(g.shape), C.c_int(len(g.shape)),
                                 _fp(a.data), _i64(a.shape), _i64(a.strides), C.c_int(len(a.shape)),
                                 _fp(b.data), _i64(b.shape), _i64(b.strides), C.c_int(len(b.shape)),
                                 _fp(da), _fp(db), C.c_int(threads or max_threads()))
    if rc:
        raise ValueError(_ERR.get(rc, str(rc)))
    return (HostTensor(da, tuple(a.shape), _row_major(a.shape)),
            HostTensor(db, tuple(b.shape), _row_major(b.shape)))


def add(a: HostTensor, b: HostTensor) -> HostTensor:
    """ops/elementwise.rs:62-73 (broadcast add; the Linear bias add)."""
    a, b = contiguous(a), contiguous(b)
    oshape = _bshape(a.shape, b.shape)
    out = np.empty(_shape_size(oshape), np.float32)
    rc = lib().oracle_add(_fp(a.data), _i64(a.shape), C.c_int(len(a.shape)),
                          _fp(b.data), _i64(b.shape), C.c_int(len(b.shape)), _fp(out))
    if rc:
        raise ValueError(_ERR.get(rc, str(rc)))
    return HostTensor(out, oshape, _row_major(oshape))


def add_backward(grad: HostTensor, a_shape: Sequence[int], b_shape: Sequence[int], threads: int = 0):
    """ops/elementwise.rs:199-211 -> (grad_a, grad_b)."""
    g = contiguous(grad)
    da = np.empty(_shape_size(a_shape), np.float32)
    db = np.empty(_shape_size(b_shape), np.float32)
    lib().oracle_add_bwd(_fp(g.data), _i64(g.shape), C.c_int(len(g.shape)),
                         _i64(a_shape), C.c_int(len(a_shape)), _i64(b_shape), C.c_int(len(b_shape)),
                         _fp(da), _fp(db), C.c_int(threads or max_threads()))
    return (HostTensor(da, tuple(a_shape), _row_major(a_shape)),
            HostTensor(db, tuple(b_shape), _row_major(b_shape)))


def bias_gelu(x: HostTensor, bias: HostTensor) -> HostTensor:
    """ops/fused.rs:251-277 (CPU backend)."""
    x, bias = contiguous(x), contiguous(bias)
    out = np.empty(_shape_size(x.shape), np.float32)
    lib().oracle_bias_gelu(_fp(x.data), _fp(bias.data), _fp(out), C.c_int64(_shape_size(x.shape)),
                           C.c_int64(x.shape[-1]))
    return HostTensor(out, tuple(x.shape), _row_major(x.shape))


def bias_gelu_backward(grad: HostTensor, x: HostTensor, bias: HostTensor):
    """ops/fused.rs:317-352 (CPU backend) -> (dx, dbias)."""
    g, x, bias = contiguous(grad), contiguous(x), contiguous(bias)
    dx = np.empty(_shape_size(x.shape), np.float32)
    db = np.empty(x.shape[-1], np.float32)
    lib().oracle_bias_gelu_bwd(_fp(g.data), _fp(x.data), _fp(bias.data), _fp(dx), _fp(db),
                               C.c_int64(_shape_size(x.shape)), C.c_int64(x.shape[-1]))
    return HostTensor(dx, tuple(x.shape), _row_major(x.shape)), HostTensor(db, (x.shape[-1],), (1,))


def adamw_step(data: np.ndarray, m: np.ndarray, v: np.ndarray, grad: np.ndarray, *, lr, beta1=0.9, beta2=0.999,
               eps=1e-8, weight_decay=0.0, step=1) -> None:
    """ops/optimizer.rs:22-65 (CPU backend), in place on flat f32 arrays."""
    lib().oracle_adamw_step(_fp(data), _fp(m), _fp(v), _fp(grad), C.c_int64(data.size), C.c_float(lr),
                            C.c_float(beta1), C.c_float(beta2), C.c_float(eps), C.c_float(weight_decay), C.c_int(step))


def powi(x: float, n: int) -> float:
    """f32::powi as ops/optimizer.rs:26-27 evaluates the bias corrections."""
    fn = lib().oracle_powi
    fn.restype = C.c_float
    return float(fn(C.c_float(x), C.c_int(n)))


def _split(shape, dim):
    d = dim + len(shape) if dim < 0 else dim
    outer = int(np.prod(shape[:d], dtype=np.int64)) if d else 1
    inner = int(np.prod(shape[d + 1:], dtype=np.int64)) if d + 1 < len(shape) else 1
    return max(outer, 1), int(shape[d]), max(inner, 1)


def softmax(a: np.ndarray, dim: int = -1) -> np.ndarray:
    """ops/norm.rs:10-50 on a C-contiguous f32 array."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty_like(a)
    outer, size, inner = _split(a.shape, dim)
    lib().oracle_softmax(_fp(a), _fp(out), C.c_int64(outer), C.c_int64(size), C.c_int64(inner))
    return out


def softmax_backward(grad: np.ndarray, sm: np.ndarray, dim: int = -1) -> np.ndarray:
    """ops/norm.rs:95-123."""
    grad = np.ascontiguousarray(grad, dtype=np.float32)
    sm = np.ascontiguousarray(sm, dtype=np.float32)
    out = np.empty_like(sm)
    outer, size, inner = _split(sm.shape, dim)
    lib().oracle_softmax_bwd(_fp(grad), _fp(sm), _fp(out), C.c_int64(outer), C.c_int64(size), C.c_int64(inner))
    return out


def _ptr_array(arrays):
    return (_f32p * len(arrays))(*[_fp(a) for a in arrays])


def grad_norm(grads) -> float:
    """ops/optimizer.rs:126-138 over a list of flat f32 arrays."""
    fn = lib().oracle_grad_norm
    fn.restype = C.c_float
    sizes = (C.c_int64 * len(grads))(*[g.size for g in grads])
    return float(fn(_ptr_array(grads), sizes, C.c_int(len(grads))))


def clip_and_step(params, ms, vs, grads, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1,
                  max_grad_norm=0.0) -> float:
    """ops/optimizer.rs:226-245 (CPU backend), in place on lists of flat f32 arrays; returns the norm."""
    fn = lib().oracle_clip_and_step
    fn.restype = C.c_float
    sizes = (C.c_int64 * len(params))(*[p.size for p in params])
    return float(fn(_ptr_array(params), _ptr_array(ms), _ptr_array(vs), _ptr_array(grads), sizes,
                    C.c_int(len(params)), C.c_float(lr), C.c_float(beta1), C.c_float(beta2), C.c_float(eps),
                    C.c_float(weight_decay), C.c_int(step), C.c_float(max_grad_norm)))


def matmul_contig_raw(a: np.ndarray, b: np.ndarray, out: np.ndarray, batch: int, a_batch: int,
                      b_batch: int, m: int, k: int, n: int, threads: int) -> None:
    """The bare loop nest of ops/matmul.rs:54-70 on caller-owned buffers (bench baseline)."""
    lib().oracle_matmul_contig(_fp(a), _fp(b), _fp(out), C.c_int64(batch), C.c_int64(a_batch),
                               C.c_int64(b_batch), C.c_int64(m), C.c_int64(k), C.c_int64(n),
                               C.c_int(threads))
