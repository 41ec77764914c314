"""ctypes binding of ``libmni_b200.so`` -- the same C ABI the reference's Rust shim binds.

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH, source_hash

MAX_DIMS = 8

PRECISION_TF32 = 1 << 0
ACCUMULATE_C = 1 << 1
ACCUMULATE_DA = 1 << 2
ACCUMULATE_DB = 1 << 3
ACCUMULATE_DBIAS = 1 << 4
FORCE_TENSOR_PATH = 1 << 8
FORCE_SKINNY_PATH = 1 << 9
FORCE_PACK = 1 << 10


def force_split_k(s: int) -> int:
    return (int(s) & 0xFF) << 16


STATUS_NAMES = {
    0: "OK", 1: "ERR_NDIM", 2: "ERR_INNER_DIM", 3: "ERR_BROADCAST", 4: "ERR_ARG", 5: "ERR_DEVICE",
    6: "ERR_CUDA", 7: "ERR_WORKSPACE", 8: "ERR_TIMEOUT", 9: "ERR_TOO_LARGE",
}


class View(C.Structure):
    """``mni_b200_view``: pointer + shape + element strides of one tensor."""
    _fields_ = [("ptr", C.c_void_p), ("ndim", C.c_int32),
                ("shape", C.c_int64 * MAX_DIMS), ("stride", C.c_int64 * MAX_DIMS)]


class MniError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"mni_b200 {STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message


_lib = None

_SIGNATURES = {
    "mni_b200_version": (C.c_int, []),
    "mni_b200_build_id": (C.c_char_p, []),
    "mni_b200_last_error": (C.c_char_p, []),
    "mni_b200_matmul_fwd": (C.c_int, [C.POINTER(View), C.POINTER(View), C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "mni_b200_matmul_bias_gelu_fwd": (C.c_int, [C.POINTER(View), C.POINTER(View), C.c_void_p, C.c_void_p, C.c_void_p,
                                                C.c_uint32, C.c_void_p]),
    "mni_b200_matmul_bwd": (C.c_int, [C.POINTER(View), C.POINTER(View), C.POINTER(View), C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_uint32, C.c_void_p]),
    "mni_b200_add_bias": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "mni_b200_add_bias_bwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_uint32, C.c_void_p]),
    "mni_b200_add_bias_bwd_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_uint32,
                                                C.c_void_p]),
    "mni_b200_bias_gelu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "mni_b200_bias_gelu_bwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                         C.c_int64, C.c_uint32, C.c_void_p]),
    "mni_b200_softmax_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "mni_b200_softmax_bwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                       C.c_void_p]),
    "mni_b200_grad_sumsq": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_uint32, C.c_void_p]),
    "mni_b200_adamw_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_float,
                                      C.c_float, C.c_float, C.c_float, C.c_uint32, C.c_void_p, C.c_float, C.c_int,
                                      C.c_void_p]),
    "mni_b200_contiguous": (C.c_int, [C.POINTER(View), C.c_void_p, C.c_void_p]),
    "mni_b200_sm_reserve": (C.c_int, [C.c_int]),
    "mni_b200_workspace_set": (C.c_int, [C.c_void_p, C.c_size_t]),
    "mni_b200_workspace_query": (C.c_int, [C.POINTER(View), C.POINTER(View), C.c_uint32, C.POINTER(C.c_size_t)]),
    "mni_b200_plan_describe": (C.c_int, [C.POINTER(View), C.POINTER(View), C.c_int, C.c_uint32, C.c_int, C.c_char_p,
                                         C.c_size_t]),
    "mni_b200_device_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "mni_b200_launch_count": (C.c_uint64, []),
    "mni_b200_release": (C.c_int, []),
    "mni_b200_role_wait_cycles": (C.c_int, [C.POINTER(C.c_uint64), C.c_int]),
}


def exported_symbols() -> list:
    return sorted(_SIGNATURES)


def lib() -> C.CDLL:
    """Loads the in-tree shared library.  Raises if it has not been built, or if it was built from
    sources that differ from the tree's (the library carries a hash of its sources)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m framework_b200.build` "
                "(there is no CPU or library fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        built_from = handle.mni_b200_build_id().decode()
        if built_from != source_hash():
            raise ImportError(
                f"{LIB_PATH} was built from other sources than the ones in csrc/ and include/ "
                "(rebuild it with `python -m framework_b200.build`); refusing to run a stale library")
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise MniError(status, lib().mni_b200_last_error().decode("utf-8", "replace"))


def make_view(ptr: int, shape, strides) -> View:
    if len(shape) > MAX_DIMS:
        raise MniError(4, f"{len(shape)} dims exceed the ABI's {MAX_DIMS}")
    v = View()
    v.ptr = ptr
    v.ndim = len(shape)
    for i, (s, t) in enumerate(zip(shape, strides)):
        v.shape[i] = int(s)
        v.stride[i] = int(t)
    return v
