"""
attorch_b200: the fused linear layer of BobMcDear/attorch (``attorch.Linear``), rebuilt for NVIDIA
B200 (sm_100a) as hand-written tcgen05 / TMA / TMEM CUDA kernels behind a C ABI.

Public surface (mirrors the reference's for this path, attorch/__init__.py:7-22):
    Linear            drop-in for attorch.Linear
    LinearAutoGrad    the autograd function behind it
    check_status      raise if a kernel reported a device-side time-out
    Sigmoid ... Softshrink, ActFuncAutoGrad
                      the standalone activation layers with fused dropout (attorch/act_layers.py)
    GLU, GLUAutoGrad  the gated linear unit with an arbitrary activation (attorch/glu_layer.py)
    GatedLinear       a projection with the gated linear unit fused into its epilogue
    CrossEntropyLoss, CrossEntropyLossAutoGrad
                      mean cross-entropy over class indices (attorch/cross_entropy_loss_layer.py)
    LayerNorm, LayerNormAutoGrad
                      layer normalisation (attorch/layer_norm_layer.py)
    LayerNormLinear   a LayerNorm and the Linear after it with no cast pass between them
    set_dropout_stream
                      the reference's dropout mask (default) or a cheaper generator
    nn                torch.nn with this package's modules in place of PyTorch's (attorch/nn.py)
    convert           parameters between torch.nn.Linear's [out, in] and this package's [in, out]
"""

from . import convert, nn
from .act_layers import (CELU, ELU, GELU, SELU, ActFuncAutoGrad, Hardshrink, Hardsigmoid, Hardswish,
                         Hardtanh, LeakyReLU, LogSigmoid, Mish, ReLU, ReLU6, Sigmoid, SiLU, Softplus,
                         Softshrink, Softsign, Tanh, Tanhshrink, set_dropout_stream)
from .cross_entropy_loss_layer import CrossEntropyLoss, CrossEntropyLossAutoGrad
from .gated_linear import GatedLinear, GatedLinearAutoGrad
from .glu_layer import GLU, GLUAutoGrad
from .layer_norm_layer import LayerNorm, LayerNormAutoGrad, LayerNormLinear
from .linear_layer import (Linear, LinearAutoGrad, check_status, get_output_dtype, set_gemm_flags,
                           set_reserved_sms, set_save_derivative)

__all__ = ['convert', 'nn', 'CrossEntropyLoss', 'CrossEntropyLossAutoGrad', 'GatedLinear', 'GatedLinearAutoGrad', 'GLU', 'GLUAutoGrad', 'LayerNorm', 'LayerNormAutoGrad', 'LayerNormLinear', 'Linear', 'LinearAutoGrad', 'check_status', 'get_output_dtype', 'set_gemm_flags',
           'set_save_derivative', 'set_reserved_sms', 'set_dropout_stream', 'ActFuncAutoGrad', 'CELU', 'ELU', 'GELU', 'SELU', 'Hardshrink',
           'Hardsigmoid', 'Hardswish', 'Hardtanh', 'LeakyReLU', 'LogSigmoid', 'Mish', 'ReLU', 'ReLU6',
           'Sigmoid', 'SiLU', 'Softplus', 'Softshrink', 'Softsign', 'Tanh', 'Tanhshrink']
