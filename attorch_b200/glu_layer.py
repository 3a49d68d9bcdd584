"""
Gated linear unit with an arbitrary activation function: drop-in replacement for the reference's
``attorch.GLU`` / ``GLUAutoGrad`` (attorch/glu_layer.py:19-138) on top of the C-ABI entry points
``ab200_glu_forward`` / ``ab200_glu_backward``.

Same constructor (``dim``, ``act_func`` with the same strings as the linear layer, default
``'sigmoid'``) and behaviour: the input is split in two along ``dim`` (whose extent must be even),
the output is ``x1 * act(x2)`` in the input's dtype.  Unlike the reference no contiguous copies of
the halves are made and the input gradient is written in one piece.
"""

from typing import Optional, Tuple

import torch
from torch import Tensor, nn

from . import _lib
from .acts import act_id, parse_act_func
from .linear_layer import _dtype_id, _require_cuda


def _outer_inner(shape: torch.Size, dim: int) -> Tuple[int, int]:
    outer = 1
    for extent in shape[:dim]:
        outer *= extent
    inner = shape[dim] // 2
    for extent in shape[dim + 1:]:
        inner *= extent
    return outer, inner


class GLUAutoGrad(torch.autograd.Function):
    """
    Autodiff for the gated linear unit; same contract as the reference's ``GLUAutoGrad``
    (attorch/glu_layer.py:19-116): ``apply(input, dim, act_func)``.
    """
    @staticmethod
    def forward(ctx, input: Tensor, dim: int, act_func: str) -> Tensor:
        name, param = parse_act_func(act_func)
        _require_cuda(input, 'input')
        dim = dim % input.ndim if input.ndim else dim
        if input.shape[dim] % 2 != 0:
            # torch.chunk would hand the reference halves of unequal size, which its kernel cannot gate.
            raise RuntimeError(f'Halving dimension must be even, but dimension {dim} is size {input.shape[dim]}')
        ctx.act = act_id(name)
        ctx.param = 0.0 if param is None else param
        ctx.dim = dim

        contiguous_input = input.contiguous()
        outer, inner = _outer_inner(input.shape, dim)
        ctx.outer, ctx.inner = outer, inner
        if input.requires_grad:
            ctx.save_for_backward(contiguous_input)

        output_shape = list(input.shape)
        output_shape[dim] //= 2
        output = torch.empty(output_shape, device=input.device, dtype=input.dtype)
        with torch.cuda.device(input.device):
            _lib.check(_lib.load().ab200_glu_forward(
                contiguous_input.data_ptr(), output.data_ptr(), outer, inner, _dtype_id(input.dtype),
                ctx.act, ctx.param, torch.cuda.current_stream().cuda_stream), 'ab200_glu_forward')
        return output

    @staticmethod
    def backward(ctx, output_grad: Tensor) -> Tuple[Optional[Tensor], ...]:
        (input,) = ctx.saved_tensors
        output_grad = output_grad.to(input.dtype).contiguous()
        input_grad = torch.empty_like(input)
        with torch.cuda.device(input.device):
            _lib.check(_lib.load().ab200_glu_backward(
                output_grad.data_ptr(), input.data_ptr(), input_grad.data_ptr(), ctx.outer, ctx.inner,
                _dtype_id(input.dtype), ctx.act, ctx.param, torch.cuda.current_stream().cuda_stream),
                'ab200_glu_backward')
        return input_grad, None, None


class GLU(nn.GLU):
    """
    Applies the gated linear unit with an arbitrary activation function to the input
    (attorch/glu_layer.py:119-138).

    Args:
        dim: Dimension over which to gate.
        act_func: Name of activation function to apply; same options as ``Linear``.
    """
    def __init__(self, dim: int = -1, act_func: str = 'sigmoid') -> None:
        super().__init__(dim)
        self.act_func = act_func

    def forward(self, input: Tensor) -> Tensor:
        return GLUAutoGrad.apply(input, self.dim, self.act_func)
