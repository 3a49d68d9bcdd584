"""
Standalone activation layers with fused dropout: drop-in replacements for the reference's
``attorch.Sigmoid`` ... ``attorch.Hardshrink`` (attorch/act_layers.py:20-570) on top of the C-ABI
entry points ``ab200_act_forward`` / ``ab200_act_input_grad``.

Same constructors (``drop_p`` and, where the PyTorch base class has them, ``inplace`` and the
activation's parameter), same behaviour: the output has the input's shape and dtype, dropout is
applied after the activation while ``training`` and ``drop_p > 0``, the seed is drawn with
``random.randint(0, 65535)`` per forward call, and backward regenerates the mask from the seed.
The mask is the reference's own: the same seed (hence the same ``random.seed``) drops the same
elements as ``tl.rand`` does there (attorch/dropout_kernels.py:26).  ``set_dropout_stream('packed')``
switches to a generator that does a quarter of the integer work and yields a different mask.
"""

import warnings
from random import randint
from typing import Optional, Tuple

import torch
from torch import Tensor, nn

from . import _lib
from .acts import act_id, parse_act_func
from .linear_layer import _dtype_id, _require_cuda


_dropout_flags = 0


def set_dropout_stream(stream: str) -> None:
    """
    Chooses the generator behind the dropout mask of layers called from now on: ``'reference'``
    (default; bit-identical to the reference's mask for a given seed, one Philox block per element)
    or ``'packed'`` (one Philox block per four elements; faster on 2-byte tensors, other mask).
    """
    global _dropout_flags
    if stream not in ('reference', 'packed'):
        raise ValueError(f"dropout stream must be 'reference' or 'packed', received {stream!r}")
    _dropout_flags = _lib.FLAG_DROPOUT_PACKED if stream == 'packed' else 0


class ActFuncAutoGrad(torch.autograd.Function):
    """
    Autodiff for activation functions; same contract as the reference's ``ActFuncAutoGrad``
    (attorch/act_layers.py:20-117): ``apply(input, act_func, drop_p, training)``.
    """
    @staticmethod
    def forward(ctx, input: Tensor, act_func: str, drop_p: float, training: bool) -> Tensor:
        name, param = parse_act_func(act_func)
        _require_cuda(input, 'input')
        ctx.act = act_id(name)
        ctx.param = 0.0 if param is None else param
        ctx.drop_p = float(drop_p)
        ctx.dropout = drop_p > 0 and training
        ctx.seed = randint(0, 65535) if ctx.dropout else 0
        ctx.flags = _dropout_flags
        if input.requires_grad:
            ctx.save_for_backward(input)

        flattened_input = input.contiguous().view(-1)
        output = torch.empty_like(flattened_input)
        with torch.cuda.device(input.device):
            _lib.check(_lib.load().ab200_act_forward(
                flattened_input.data_ptr(), output.data_ptr(), flattened_input.numel(),
                _dtype_id(input.dtype), ctx.act, ctx.param, ctx.drop_p if ctx.dropout else 0.0,
                ctx.seed, torch.cuda.current_stream().cuda_stream, ctx.flags), 'ab200_act_forward')
        return output.view(input.shape)

    @staticmethod
    def backward(ctx, output_grad: Tensor) -> Tuple[Optional[Tensor], ...]:
        (input,) = ctx.saved_tensors
        flattened_input = input.contiguous().view(-1)
        output_grad = output_grad.to(input.dtype).contiguous().view(-1)
        input_grad = torch.empty_like(flattened_input)
        with torch.cuda.device(input.device):
            _lib.check(_lib.load().ab200_act_input_grad(
                output_grad.data_ptr(), flattened_input.data_ptr(), input_grad.data_ptr(),
                flattened_input.numel(), _dtype_id(input.dtype), ctx.act, ctx.param,
                ctx.drop_p if ctx.dropout else 0.0, ctx.seed,
                torch.cuda.current_stream().cuda_stream, ctx.flags), 'ab200_act_input_grad')
        return input_grad.view(input.shape), None, None, None


def _warn_inplace(inplace: bool, name: str) -> None:
    if inplace is True:
        warnings.warn(f'In-place {name} currently not supported; falling back to out-of-place.')


class Sigmoid(nn.Sigmoid):
    """Applies sigmoid to the input, optionally fusing dropout (attorch/act_layers.py:120-135)."""
    def __init__(self, drop_p: float = 0.0) -> None:
        super().__init__()
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'sigmoid', self.drop_p, self.training)


class LogSigmoid(nn.LogSigmoid):
    """Applies the log of sigmoid, optionally fusing dropout."""
    def __init__(self, drop_p: float = 0.0) -> None:
        super().__init__()
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'logsigmoid', self.drop_p, self.training)


class Tanh(nn.Tanh):
    """Applies tanh, optionally fusing dropout."""
    def __init__(self, drop_p: float = 0.0) -> None:
        super().__init__()
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'tanh', self.drop_p, self.training)


class ReLU(nn.ReLU):
    """Applies ReLU, optionally fusing dropout."""
    def __init__(self, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(inplace=False)
        _warn_inplace(inplace, 'ReLU')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'relu', self.drop_p, self.training)


class GELU(nn.GELU):
    """Applies GELU (exact or tanh approximation), optionally fusing dropout."""
    def __init__(self, approximate: str = 'none', drop_p: float = 0.0) -> None:
        if approximate not in ['none', 'tanh']:
            raise RuntimeError(f'Approximation algorithm {approximate} invalid.')
        super().__init__(approximate=approximate)
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'gelu' if self.approximate == 'none' else 'geluapprox',
                                     self.drop_p, self.training)


class SiLU(nn.SiLU):
    """Applies SiLU, optionally fusing dropout."""
    def __init__(self, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(inplace=False)
        _warn_inplace(inplace, 'SiLU')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'silu', self.drop_p, self.training)


class ReLU6(nn.ReLU6):
    """Applies ReLU6, optionally fusing dropout."""
    def __init__(self, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(inplace=False)
        _warn_inplace(inplace, 'ReLU6')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'relu6', self.drop_p, self.training)


class Hardsigmoid(nn.Hardsigmoid):
    """Applies hard sigmoid, optionally fusing dropout."""
    def __init__(self, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(inplace=False)
        _warn_inplace(inplace, 'hard sigmoid')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'hardsigmoid', self.drop_p, self.training)


class Hardtanh(nn.Hardtanh):
    """Applies hard tanh (limits -1 and 1 only, as in the reference), optionally fusing dropout."""
    def __init__(self, min_val: float = -1.0, max_val: float = 1.0, inplace: bool = False,
                 drop_p: float = 0.0) -> None:
        if min_val != -1.0:
            raise RuntimeError('Hard tanh only supports a minimum value of -1.')
        if max_val != 1.0:
            raise RuntimeError('Hard tanh only supports a maximum value of -1.')
        super().__init__(inplace=False)
        _warn_inplace(inplace, 'hard tanh')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'hardtanh', self.drop_p, self.training)


class Hardswish(nn.Hardswish):
    """Applies hard Swish, optionally fusing dropout."""
    def __init__(self, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(inplace=False)
        _warn_inplace(inplace, 'hard Swish')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'hardswish', self.drop_p, self.training)


class SELU(nn.SELU):
    """Applies SELU, optionally fusing dropout."""
    def __init__(self, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(inplace=False)
        _warn_inplace(inplace, 'SELU')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'selu', self.drop_p, self.training)


class Mish(nn.Mish):
    """Applies Mish, optionally fusing dropout."""
    def __init__(self, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(inplace=False)
        _warn_inplace(inplace, 'Mish')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'mish', self.drop_p, self.training)


class Softplus(nn.Softplus):
    """Applies softplus (beta = 1, no threshold), optionally fusing dropout."""
    def __init__(self, drop_p: float = 0.0) -> None:
        super().__init__()
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'softplus', self.drop_p, self.training)


class Softsign(nn.Softsign):
    """Applies softsign, optionally fusing dropout."""
    def __init__(self, drop_p: float = 0.0) -> None:
        super().__init__()
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'softsign', self.drop_p, self.training)


class Tanhshrink(nn.Tanhshrink):
    """Applies tanh shrink, optionally fusing dropout."""
    def __init__(self, drop_p: float = 0.0) -> None:
        super().__init__()
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'tanhshrink', self.drop_p, self.training)


class LeakyReLU(nn.LeakyReLU):
    """Applies leaky ReLU, optionally fusing dropout."""
    def __init__(self, negative_slope: float = 1e-2, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(negative_slope=negative_slope, inplace=False)
        _warn_inplace(inplace, 'leaky ReLU')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'leaky_relu_' + str(self.negative_slope), self.drop_p,
                                     self.training)


class ELU(nn.ELU):
    """Applies ELU, optionally fusing dropout."""
    def __init__(self, alpha: float = 1.0, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(alpha, inplace=False)
        _warn_inplace(inplace, 'ELU')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'elu_' + str(self.alpha), self.drop_p, self.training)


class CELU(nn.CELU):
    """Applies CELU, optionally fusing dropout."""
    def __init__(self, alpha: float = 1.0, inplace: bool = False, drop_p: float = 0.0) -> None:
        super().__init__(alpha, inplace=False)
        _warn_inplace(inplace, 'CELU')
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'celu_' + str(self.alpha), self.drop_p, self.training)


class Hardshrink(nn.Hardshrink):
    """Applies hard shrink, optionally fusing dropout."""
    def __init__(self, lambd: float = 0.5, drop_p: float = 0.0) -> None:
        super().__init__(lambd)
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'hardshrink_' + str(self.lambd), self.drop_p, self.training)


class Softshrink(nn.Softshrink):
    """Applies soft shrink, optionally fusing dropout."""
    def __init__(self, lambd: float = 0.5, drop_p: float = 0.0) -> None:
        super().__init__(lambd)
        self.drop_p = drop_p

    def forward(self, input: Tensor) -> Tensor:
        return ActFuncAutoGrad.apply(input, 'softshrink_' + str(self.lambd), self.drop_p, self.training)
