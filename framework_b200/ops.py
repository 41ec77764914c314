"""Host-side mirror of the reference's operator interface for the matmul path.

Names, argument meaning and error behaviour follow src/native/src/ops/matmul.rs
and the bias branch of src/native/src/ops/elementwise.rs; every function is a thin
call into the C ABI of ``libmni_b200.so``.  Outputs are allocated here the way the
reference's ``store.zeros`` does (uninitialised memory is fine: the kernels
overwrite every element).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

from . import _lib
from .tensor import DeviceTensor, current_stream, row_major_strides, shape_size


def broadcast_shape(a: Sequence[int], b: Sequence[int]) -> tuple:
    """utils.rs:3-20.  Raises where the reference panics."""
    nd = max(len(a), len(b))
    out = []
    for i in range(nd):
        da = 1 if i < nd - len(a) else a[i - (nd - len(a))]
        db = 1 if i < nd - len(b) else b[i - (nd - len(b))]
        if da == db:
            out.append(da)
        elif da == 1:
            out.append(db)
        elif db == 1:
            out.append(da)
        else:
            raise ValueError(f"shapes {list(a)} and {list(b)} are not broadcastable")
    return tuple(out)


def _matmul_out_shape(a: DeviceTensor, b: DeviceTensor) -> tuple:
    if a.ndim < 2 or b.ndim < 2:
        raise ValueError("matmul requires at least 2D tensors")          # ops/matmul.rs:89
    if a.shape[-1] != b.shape[-2]:
        raise ValueError(f"matmul inner dimensions must match: {a.shape[-1]} vs {b.shape[-2]}")  # :94
    return broadcast_shape(a.shape[:-2], b.shape[:-2]) + (a.shape[-2], b.shape[-1])


def matmul(a: DeviceTensor, b: DeviceTensor, bias: Optional[DeviceTensor] = None, *, flags: int = 0,
           out: Optional[DeviceTensor] = None) -> DeviceTensor:
    """``ops::matmul::matmul`` (ops/matmul.rs:83-197).  ``bias`` fuses the Linear bias add."""
    oshape = _matmul_out_shape(a, b)
    if bias is not None and (bias.ndim != 1 or bias.shape[0] != oshape[-1] or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous [N] vector")
    if out is None:
        out = DeviceTensor.empty(oshape, a.storage.device)
    elif out.shape != oshape or not out.is_contiguous():
        raise ValueError("out must be contiguous with the broadcast output shape")
    va, vb = a.view_struct(), b.view_struct()
    _lib.check(_lib.lib().mni_b200_matmul_fwd(va, vb, out.ptr, bias.ptr if bias is not None else None,
                                              flags, current_stream()))
    return out


def matmul_backward(grad: DeviceTensor, a: DeviceTensor, b: DeviceTensor, *, flags: int = 0,
                    need_da: bool = True, need_db: bool = True, want_dbias: bool = False,
                    da: Optional[DeviceTensor] = None, db: Optional[DeviceTensor] = None,
                    dbias: Optional[DeviceTensor] = None):
    """``ops::matmul::matmul_backward`` (ops/matmul.rs:225-255) -> (grad_a, grad_b[, dbias])."""
    oshape = _matmul_out_shape(a, b)
    if grad.shape != oshape:
        raise ValueError(f"grad has shape {grad.shape}, forward output is {oshape}")
    dev = a.storage.device
    if need_da and da is None:
        da = DeviceTensor.empty(a.shape, dev)
    if need_db and db is None:
        db = DeviceTensor.empty(b.shape, dev)
    if want_dbias and dbias is None:
        dbias = DeviceTensor.empty((oshape[-1],), dev)
    va, vb, vg = a.view_struct(), b.view_struct(), grad.view_struct()
    _lib.check(_lib.lib().mni_b200_matmul_bwd(
        va, vb, vg, da.ptr if need_da else None, db.ptr if need_db else None,
        dbias.ptr if want_dbias else None, flags, current_stream()))
    if want_dbias:
        return da, db, dbias
    return da, db


def add(a: DeviceTensor, b: DeviceTensor) -> DeviceTensor:
    """Bias branch of ``ops::elementwise::add`` (ops/elementwise.rs:105-130): [.., N] + [N]."""
    if not (b.ndim == 1 and a.ndim >= 1 and a.shape[-1] == b.shape[0]):
        raise NotImplementedError("only the Linear bias add ([..., N] + [N]) is on this path")
    a = a.contiguous()
    b = b.contiguous()
    out = DeviceTensor.empty(a.shape, a.storage.device)
    n = a.shape[-1]
    rows = shape_size(a.shape[:-1])
    _lib.check(_lib.lib().mni_b200_add_bias(a.ptr, b.ptr, out.ptr, rows, n, current_stream()))
    return out


def add_backward(grad: DeviceTensor, a_shape: Sequence[int], b_shape: Sequence[int], *,
                 flags: int = 0) -> Tuple[DeviceTensor, DeviceTensor]:
    """``add_backward`` for the bias branch (ops/elementwise.rs:213-231) -> (grad_a, grad_bias)."""
    if tuple(grad.shape) != tuple(a_shape) or len(b_shape) != 1 or b_shape[0] != grad.shape[-1]:
        raise NotImplementedError("only the Linear bias add ([..., N] + [N]) is on this path")
    g = grad.contiguous()
    ga = DeviceTensor.empty(a_shape, g.storage.device)
    gb = DeviceTensor.empty(b_shape, g.storage.device)
    n = g.shape[-1]
    rows = shape_size(g.shape[:-1])
    _lib.check(_lib.lib().mni_b200_add_bias_bwd(g.ptr, ga.ptr, gb.ptr, rows, n, flags, current_stream()))
    return ga, gb


def bias_gelu(x: DeviceTensor, bias: DeviceTensor) -> DeviceTensor:
    """``ops::fused::bias_gelu`` (ops/fused.rs:279-314): gelu(x + bias) with bias over the last dim."""
    if bias.ndim != 1 or x.ndim < 1 or x.shape[-1] != bias.shape[0]:
        raise ValueError("bias must be a [C] vector matching x's last dim")
    x, bias = x.contiguous(), bias.contiguous()
    out = DeviceTensor.empty(x.shape, x.storage.device)
    n = x.shape[-1]
    _lib.check(_lib.lib().mni_b200_bias_gelu(x.ptr, bias.ptr, out.ptr, shape_size(x.shape[:-1]), n, current_stream()))
    return out


def bias_gelu_backward(grad: DeviceTensor, x: DeviceTensor, bias: DeviceTensor, *,
                       flags: int = 0) -> Tuple[DeviceTensor, DeviceTensor]:
    """``ops::fused::bias_gelu_backward`` (ops/fused.rs:354-392) -> (dx, dbias)."""
    if tuple(grad.shape) != tuple(x.shape) or bias.shape != (x.shape[-1],):
        raise ValueError("grad must have x's shape and bias must be [C]")
    g, x, bias = grad.contiguous(), x.contiguous(), bias.contiguous()
    dx = DeviceTensor.empty(x.shape, x.storage.device)
    dbias = DeviceTensor.empty(bias.shape, x.storage.device)
    n = x.shape[-1]
    _lib.check(_lib.lib().mni_b200_bias_gelu_bwd(g.ptr, x.ptr, bias.ptr, dx.ptr, dbias.ptr,
                                                 shape_size(x.shape[:-1]), n, flags, current_stream()))
    return dx, dbias


def matmul_bias_gelu(a: DeviceTensor, b: DeviceTensor, bias: DeviceTensor, *, flags: int = 0,
                     want_pre: bool = True) -> Tuple[Optional[DeviceTensor], DeviceTensor]:
    """matmul followed by bias_gelu in one GEMM launch -> (pre = a.b or None, out = gelu(pre + bias))."""
    oshape = _matmul_out_shape(a, b)
    if bias.ndim != 1 or bias.shape[0] != oshape[-1] or not bias.is_contiguous():
        raise ValueError("bias must be a contiguous [N] vector")
    dev = a.storage.device
    pre = DeviceTensor.empty(oshape, dev) if want_pre else None
    out = DeviceTensor.empty(oshape, dev)
    va, vb = a.view_struct(), b.view_struct()
    _lib.check(_lib.lib().mni_b200_matmul_bias_gelu_fwd(va, vb, bias.ptr, pre.ptr if pre is not None else None,
                                                        out.ptr, flags, current_stream()))
    return pre, out


def _softmax_split(shape: Sequence[int], dim: int) -> Tuple[int, int, int]:
    d = dim + len(shape) if dim < 0 else dim
    if not 0 <= d < len(shape):
        raise IndexError(f"softmax dim {dim} out of range for shape {tuple(shape)}")
    return max(shape_size(shape[:d]), 1) if d else 1, shape[d], max(shape_size(shape[d + 1:]), 1)


def softmax(a: DeviceTensor, dim: int = -1) -> DeviceTensor:
    """``ops::norm::softmax`` (ops/norm.rs:52-89).  A strided input is gathered first, as the reference's
    ``dev_ptr`` read assumes row-major data."""
    a = a if a.is_contiguous() else a.contiguous()
    outer, size, inner = _softmax_split(a.shape, dim)
    out = DeviceTensor.empty(a.shape, a.storage.device)
    _lib.check(_lib.lib().mni_b200_softmax_fwd(a.ptr, out.ptr, outer, size, inner, current_stream()))
    return out


def softmax_backward(grad: DeviceTensor, out: DeviceTensor, dim: int = -1) -> DeviceTensor:
    """``ops::norm::softmax_backward`` (ops/norm.rs:125-163) from the saved forward output."""
    if tuple(grad.shape) != tuple(out.shape):
        raise ValueError("grad and out must have the same shape")
    grad = grad if grad.is_contiguous() else grad.contiguous()
    out = out if out.is_contiguous() else out.contiguous()
    outer, size, inner = _softmax_split(out.shape, dim)
    dx = DeviceTensor.empty(out.shape, out.storage.device)
    _lib.check(_lib.lib().mni_b200_softmax_bwd(grad.ptr, out.ptr, dx.ptr, outer, size, inner, current_stream()))
    return dx


def _grad_sumsq(grads: Sequence[DeviceTensor]) -> "torch.Tensor":
    """Squared global gradient norm as a one-element f64 device tensor (no host read)."""
    import torch
    sumsq = torch.empty(1, dtype=torch.float64, device=grads[0].storage.device)
    for i, g in enumerate(grads):
        if not g.is_contiguous():
            raise ValueError("gradients must be contiguous")
        flags = _lib.ACCUMULATE_C if i else 0
        _lib.check(_lib.lib().mni_b200_grad_sumsq(g.ptr, g.size, sumsq.data_ptr(), flags, current_stream()))
    return sumsq


def grad_norm(grads: Sequence[DeviceTensor]) -> float:
    """``ops::optimizer::grad_norm`` (ops/optimizer.rs:126-171): sqrt of the f64 sum of squares, as f32."""
    if not grads:
        return 0.0
    import numpy as np
    return float(np.sqrt(np.float32(_grad_sumsq(grads).item())))


def adamw_step(param: DeviceTensor, m: DeviceTensor, v: DeviceTensor, grad: DeviceTensor, *, lr: float,
               beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0,
               step: int = 1, grad_sumsq=None, max_grad_norm: float = 0.0, write_clipped_grad: bool = True) -> None:
    """``ops::optimizer::adamw_step`` for one parameter (ops/optimizer.rs:67-120): in-place update.
    ``grad_sumsq`` (a one-element f64 device tensor) with ``max_grad_norm`` > 0 applies the clip of
    ``clip_and_step`` inside the same pass."""
    if not (param.is_contiguous() and m.is_contiguous() and v.is_contiguous() and grad.is_contiguous()):
        raise ValueError("adamw_step needs contiguous tensors")
    if not (param.size == m.size == v.size == grad.size):
        raise ValueError("param, m, v and grad must have the same size")
    sq = grad_sumsq.data_ptr() if grad_sumsq is not None else None
    _lib.check(_lib.lib().mni_b200_adamw_step(param.ptr, m.ptr, v.ptr, grad.ptr, param.size, lr, beta1, beta2, eps,
                                              weight_decay, int(step), sq, max_grad_norm,
                                              1 if write_clipped_grad else 0, current_stream()))


def clip_and_step(params: Sequence[DeviceTensor], ms: Sequence[DeviceTensor], vs: Sequence[DeviceTensor],
                  grads: Sequence[DeviceTensor], *, lr: float, beta1: float = 0.9, beta2: float = 0.999,
                  eps: float = 1e-8, weight_decay: float = 0.0, step: int = 1, max_grad_norm: float = 0.0) -> float:
    """``ops::optimizer::clip_and_step`` (ops/optimizer.rs:247-276): global-norm clip and AdamW over all
    parameters; returns the norm before clipping.  The norm stays on the device until every step kernel is
    queued; the read that returns it is the call's only synchronisation."""
    if not params:
        return 0.0
    import numpy as np
    sumsq = _grad_sumsq(grads)
    for p, m, v, g in zip(params, ms, vs, grads):
        adamw_step(p, m, v, g, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, step=step,
                   grad_sumsq=sumsq, max_grad_norm=max_grad_norm)
    return float(np.sqrt(np.float32(sumsq.item())))


def permute(a: DeviceTensor, dims: Sequence[int]) -> DeviceTensor:
    """``ops::layout::permute``: a stride-only view sharing the storage (what the reference's CPU backend
    does, ops/layout.rs:112-134); the matmul kernels read it in place."""
    return a.permute(dims)


def permute_backward(grad: DeviceTensor, dims: Sequence[int], orig_shape: Sequence[int]) -> DeviceTensor:
    """``ops::layout::permute_backward`` (ops/layout.rs:198-212): the gradient of the permuted tensor, put
    back into the original layout -- one device gather of the inverse-permuted view."""
    if tuple(grad.shape) != tuple(orig_shape[d] for d in dims):
        raise ValueError(f"grad has shape {grad.shape}, expected {tuple(orig_shape[d] for d in dims)}")
    inv = [0] * len(dims)
    for i, d in enumerate(dims):
        inv[d] = i
    return grad.permute(inv).contiguous()


class Linear:
    """``Linear`` of src/nn.ts:8-26 over device tensors: y = x.W + b with W [in, out].

    ``forward`` runs the drop-in sequence (matmul, then the stand-alone bias add, the
    two N-API calls of nn.ts:24); ``forward_fused`` folds the bias into the GEMM epilogue.
    """

    def __init__(self, weight: DeviceTensor, bias: DeviceTensor):
        if weight.ndim != 2 or bias.shape != (weight.shape[1],):
            raise ValueError("weight must be [in, out] and bias [out]")
        self.weight = weight
        self.bias = bias

    def forward(self, x: DeviceTensor) -> DeviceTensor:
        return add(matmul(x, self.weight), self.bias)

    def forward_fused(self, x: DeviceTensor, flags: int = 0) -> DeviceTensor:
        return matmul(x, self.weight, self.bias, flags=flags)

    def backward(self, x: DeviceTensor, dy: DeviceTensor, flags: int = 0):
        """-> (dx, dW, db): add_backward then matmul_backward, with dbias fused into one call."""
        dx, dw, dbias = matmul_backward(dy, x, self.weight, flags=flags, want_dbias=True)
        return dx, dw, dbias


def sm_reserve(sms: int) -> None:
    """Keeps `sms` SMs out of the tensor-core kernels' grids (0 = none): room for a collective that runs beside them."""
    _lib.check(_lib.lib().mni_b200_sm_reserve(int(sms)))


def device_status() -> int:
    """Synchronises the current stream; raises if a kernel recorded a bounded-wait timeout."""
    import ctypes as C
    detail = C.c_uint32(0)
    _lib.check(_lib.lib().mni_b200_device_status(current_stream(), C.byref(detail)))
    return int(detail.value)


def launch_count() -> int:
    return int(_lib.lib().mni_b200_launch_count())


def plan_describe(a_shape: Sequence[int], b_shape: Sequence[int], *, a_strides: Optional[Sequence[int]] = None,
                  b_strides: Optional[Sequence[int]] = None, backward: int = 0, flags: int = 0,
                  sm_count: int = 148) -> list:
    """The launches ``matmul`` (backward=0) or ``matmul_backward`` (1; 2 = with the bias gradient) would make for
    operands of these shapes and element strides (row-major when not given) on a device with `sm_count` SMs:
    one line of text per launch.  Needs no device -- the planner is host arithmetic."""
    import ctypes as C
    va = _lib.make_view(256, a_shape, a_strides if a_strides is not None else row_major_strides(a_shape))
    vb = _lib.make_view(256, b_shape, b_strides if b_strides is not None else row_major_strides(b_shape))
    buf = C.create_string_buffer(8192)
    _lib.check(_lib.lib().mni_b200_plan_describe(C.byref(va), C.byref(vb), int(backward), int(flags), int(sm_count),
                                                 buf, len(buf)))
    return buf.value.decode().splitlines()
