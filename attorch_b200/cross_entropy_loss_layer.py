"""
Drop-in replacement for ``attorch.CrossEntropyLoss`` (attorch/cross_entropy_loss_layer.py:20-166 of
the reference): the mean cross-entropy loss between logits ``[batch, classes]`` and class indices,
with optional class weights - the loss the final projection of a language model feeds
(examples/wikitext-2/gpt.py:116-135).  The device work runs in the library's CUDA kernels
(``ab200_cross_entropy_forward`` / ``ab200_cross_entropy_backward``); this module mirrors the
reference's host logic: argument checks, the output-dtype rule, which tensors are kept.

There is no CPU path: on a machine without the built library or without a CUDA device it raises.
"""

from typing import Optional, Tuple

import torch
from torch import Tensor, nn

from . import _lib
from .linear_layer import _dtype_id, _ptr, _require_cuda


def get_loss_dtype(input_dtype: torch.dtype) -> torch.dtype:
    """
    fp32 while CUDA autocast is enabled, else the input's dtype: the reference's
    ``get_output_dtype(input.dtype, autocast='fp32')`` (attorch/utils.py:27-60,
    attorch/cross_entropy_loss_layer.py:58).
    """
    return torch.float32 if torch.is_autocast_enabled('cuda') else input_dtype


class CrossEntropyLossAutoGrad(torch.autograd.Function):
    """
    Autodiff for the cross-entropy loss; same call contract as the reference's
    ``CrossEntropyLossAutoGrad.apply(input, target, weight)``.
    """
    @staticmethod
    def forward(ctx, input: Tensor, target: Tensor, weight: Optional[Tensor] = None) -> Tensor:
        assert input.ndim == 2, f'Inputs of rank other than 2 not valid'
        assert len(input) == len(target), \
            f'Incompatible input shape ({input.shape}) and target shape ({target.shape})'
        assert weight is None or len(weight) == input.shape[1], \
            f'Dimensionality of weight vector ({len(weight)}) and input features ({input.shape[1]}) not equal'
        _require_cuda(input, 'input')
        _require_cuda(target, 'target')

        batch_dim, feat_dim = input.shape
        output_dtype = get_loss_dtype(input.dtype)
        lib = _lib.load()
        target_op = target if (target.dtype is torch.int64 and target.is_contiguous()) else target.long().contiguous()
        weight_op = None
        if weight is not None:
            _require_cuda(weight, 'weight')
            weight_op = weight if weight.is_contiguous() else weight.contiguous()
        with torch.cuda.device(input.device):
            stream = torch.cuda.current_stream().cuda_stream
            output = torch.empty((), dtype=output_dtype, device=input.device)
            lse = torch.empty(batch_dim, dtype=torch.float32, device=input.device)
            ws_bytes = int(lib.ab200_cross_entropy_workspace_bytes(batch_dim))
            workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=input.device)
            _lib.check(lib.ab200_cross_entropy_forward(
                _ptr(input), _ptr(target_op), _ptr(weight_op), _ptr(output), _ptr(lse), batch_dim, feat_dim,
                input.stride(0), input.stride(1), _dtype_id(input.dtype),
                _dtype_id(weight_op.dtype) if weight_op is not None else 0, _dtype_id(output_dtype),
                _ptr(workspace), ws_bytes, stream), 'ab200_cross_entropy_forward')

        ctx.output_dtype = output_dtype
        ctx.has_weight = weight is not None
        if input.requires_grad:
            saved = [input, target_op, lse, workspace]
            if weight_op is not None:
                saved.append(weight_op)
            ctx.save_for_backward(*saved)
        return output

    @staticmethod
    def backward(ctx, output_grad: Tensor) -> Tuple[Optional[Tensor], ...]:
        saved = ctx.saved_tensors
        input, target, lse, workspace = saved[:4]
        weight = saved[4] if ctx.has_weight else None
        batch_dim, feat_dim = input.shape
        lib = _lib.load()
        with torch.cuda.device(input.device):
            stream = torch.cuda.current_stream().cuda_stream
            input_grad = torch.empty((batch_dim, feat_dim), dtype=ctx.output_dtype, device=input.device)
            grad = output_grad if output_grad.is_cuda else output_grad.to(input.device)
            _lib.check(lib.ab200_cross_entropy_backward(
                _ptr(grad), _dtype_id(grad.dtype), _ptr(input), _ptr(target), _ptr(weight), _ptr(lse),
                _ptr(workspace), _ptr(input_grad), batch_dim, feat_dim, input.stride(0), input.stride(1),
                feat_dim, _dtype_id(input.dtype), _dtype_id(weight.dtype) if weight is not None else 0,
                _dtype_id(ctx.output_dtype), stream), 'ab200_cross_entropy_backward')
        # One slot per forward argument (attorch/cross_entropy_loss_layer.py:116-118 pads with None).
        return input_grad, None, None


class CrossEntropyLoss(nn.CrossEntropyLoss):
    """
    Measures the mean cross entropy loss between the input and target, with optional reweighing of
    each class.  Same constructor and restrictions as the reference's ``attorch.CrossEntropyLoss``
    (attorch/cross_entropy_loss_layer.py:121-166): only ``reduction='mean'``, no ignore index, no
    label smoothing, inputs of shape ``[batch, classes]``.

    Args:
        reduction: Reduction strategy for the output. Only 'mean' is supported.
            Providing size_average and reduce overrides this argument.
        size_average: Flag for averaging instead of summing the loss entries when reduce is True.
            Only averaging is supported.
        reduce: Flag for averaging or summing all the loss entries instead of returning a loss per
            element. Only averaging is supported.
        weight: Optional class weight vector, with None for no reweighing.
        ignore_index: This argument is not supported.
        label_smoothing: This argument is not supported.
    """
    def __init__(self, reduction: str = 'mean', size_average: Optional[bool] = None,
                 reduce: Optional[bool] = None, weight: Optional[Tensor] = None,
                 ignore_index: int = -100, label_smoothing: float = 0.0) -> None:
        super().__init__(weight, size_average, ignore_index, reduce, reduction, label_smoothing)
        if self.reduction != 'mean':
            raise RuntimeError('Cross entropy only supports averaging the loss.')
        if label_smoothing > 0.0:
            raise RuntimeError('Cross entropy does not support label smoothing.')

    def forward(self, input: Tensor, target: Tensor) -> Tensor:
        return CrossEntropyLossAutoGrad.apply(input, target, self.weight)
