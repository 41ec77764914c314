"""CPU: the C-ABI library loads, exports every symbol the header declares, and rejects bad arguments
with the reference's error classes before it touches a device."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib():
    from framework_b200 import build, _lib
    build.build_library()
    return _lib.lib()


def test_header_symbols_are_exported(lib):
    from framework_b200 import _lib
    header = open(os.path.join(ROOT, "include", "mni_b200.h")).read()
    declared = sorted(set(re.findall(r"MNI_B200_API[^;(]*?\b(mni_b200_\w+)\s*\(", header)))
    assert declared, "no declarations found in include/mni_b200.h"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == _lib.exported_symbols(), "ctypes signature table and header disagree"


def test_version(lib):
    assert lib.mni_b200_version() >= 100


def _view(shape, strides=None):
    from framework_b200 import _lib
    from framework_b200.tensor import row_major_strides
    return _lib.make_view(256, shape, strides or row_major_strides(shape))


def test_argument_errors_need_no_device(lib):
    a = _view([2, 3])
    assert lib.mni_b200_matmul_fwd(a, _view([4, 2]), None, None, 0, None) == 2       # inner dims
    assert b"inner dimensions must match" in lib.mni_b200_last_error()
    assert lib.mni_b200_matmul_fwd(_view([3]), _view([3, 2]), None, None, 0, None) == 1  # ndim < 2
    assert b"at least 2D" in lib.mni_b200_last_error()
    assert lib.mni_b200_matmul_fwd(_view([2, 2, 3]), _view([3, 3, 2]), None, None, 0, None) == 3  # broadcast
    assert lib.mni_b200_matmul_fwd(None, _view([3, 2]), None, None, 0, None) == 4       # null view
    assert lib.mni_b200_matmul_bwd(a, _view([3, 2]), _view([2, 5]), None, None, None, 0, None) == 4  # dc shape
    assert lib.mni_b200_add_bias(None, None, None, -1, 4, None) == 4


def test_host_wrapper_raises_like_the_reference():
    import torch  # noqa: F401  (host-side checks run before any device call)
    from framework_b200 import ops

    class Fake:
        def __init__(self, shape):
            self.shape, self.ndim = tuple(shape), len(shape)
    with pytest.raises(ValueError, match="at least 2D"):
        ops._matmul_out_shape(Fake([3]), Fake([3, 2]))
    with pytest.raises(ValueError, match="inner dimensions must match: 3 vs 4"):
        ops._matmul_out_shape(Fake([2, 3]), Fake([4, 2]))
    with pytest.raises(ValueError, match="not broadcastable"):
        ops._matmul_out_shape(Fake([2, 2, 3]), Fake([3, 3, 2]))
    assert ops._matmul_out_shape(Fake([4, 1, 5, 3]), Fake([6, 3, 2])) == (4, 6, 5, 2)
    assert ops.broadcast_shape([], [7]) == (7,)
