"""CPU oracle for the matmul hot path -- TEST INFRASTRUCTURE ONLY.

Only tests/, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / reference
legs of ``bench.py`` may import this package.  The product (``framework_b200``)
never does.
"""
from .oracle import (  # noqa: F401
    HostTensor, build, lib, matmul, matmul_backward, add, add_backward,
    permute, permute_backward, contiguous, max_threads, matmul_contig_raw, bias_gelu, bias_gelu_backward, adamw_step, grad_norm, clip_and_step,
    softmax, softmax_backward, powi,
)
