"""B200-native matmul hot path of mni-ml/framework: Tensor.matmul forward/backward and
the Linear bias add, as hand-written sm_100a kernels behind a C ABI.

``framework_b200.csrc`` holds the CUDA sources and the C ABI implementation,
``framework_b200.ops`` the host-side mirror of the reference's operator interface.
"""
from . import _lib  # noqa: F401
from .ops import (  # noqa: F401
    Linear, adamw_step, add, add_backward, bias_gelu, bias_gelu_backward, broadcast_shape, clip_and_step,
    device_status, grad_norm, launch_count, matmul, matmul_backward, matmul_bias_gelu, permute, permute_backward,
    plan_describe, sm_reserve, softmax, softmax_backward,
)
from .tensor import DeviceTensor  # noqa: F401

__all__ = ["DeviceTensor", "Linear", "adamw_step", "add", "add_backward", "bias_gelu", "bias_gelu_backward",
           "broadcast_shape", "clip_and_step", "device_status", "grad_norm", "launch_count", "matmul", "matmul_backward", "matmul_bias_gelu", "permute", "permute_backward", "plan_describe", "sm_reserve", "softmax", "softmax_backward"]
