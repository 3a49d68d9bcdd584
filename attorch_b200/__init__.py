"""
attorch_b200: the fused linear layer of BobMcDear/attorch (``attorch.Linear``), rebuilt for NVIDIA
B200 (sm_100a) as hand-written tcgen05 / TMA / TMEM CUDA kernels behind a C ABI.

Public surface (mirrors the reference's for this path, attorch/__init__.py:7-22):
    Linear            drop-in for attorch.Linear
    LinearAutoGrad    the autograd function behind it
    check_status      raise if a kernel reported a device-side time-out
"""

from .linear_layer import (Linear, LinearAutoGrad, check_status, get_output_dtype, set_gemm_flags,
                           set_save_derivative)

__all__ = ['Linear', 'LinearAutoGrad', 'check_status', 'get_output_dtype', 'set_gemm_flags',
           'set_save_derivative']
