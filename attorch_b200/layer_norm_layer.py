"""
Drop-in replacement for ``attorch.LayerNorm`` (attorch/layer_norm_layer.py:19-213 of the reference):
layer normalisation over the last dimension with optional weight and bias, the step in front of the
first projection of a transformer block (examples/wikitext-2/gpt.py:82), and ``LayerNormLinear``, which
runs a ``LayerNorm`` and the ``Linear`` that follows it with no cast pass between them.  The device work
runs in the library's CUDA kernels (``ab200_layer_norm_forward`` / ``ab200_layer_norm_backward``); this
module mirrors the reference's host logic: flattening, the output-dtype rule, which tensors are kept.

There is no CPU path: on a machine without the built library or without a CUDA device it raises.
"""

from typing import Optional, Tuple

import torch
from torch import Tensor, nn

from . import _lib
from .linear_layer import (Linear, _dtype_id, _ptr, _require_cuda, _stream_scratch,
                           get_output_dtype as linear_output_dtype)


def get_norm_dtype(input_dtype: torch.dtype, autocast_to_fp32: bool) -> torch.dtype:
    """
    fp32 while CUDA autocast is enabled and ``autocast_to_fp32`` is set, else the input's dtype: the
    reference's ``get_output_dtype(input.dtype, autocast='fp32' if autocast_to_fp32 else None)``
    (attorch/utils.py:27-60, attorch/layer_norm_layer.py:55-56).  The reference asserts that the
    autocast dtype is fp16 or fp32; bf16 autocast is accepted here, as in the linear layer.
    """
    if torch.is_autocast_enabled('cuda') and autocast_to_fp32:
        return torch.float32
    return input_dtype


def _wider(a: torch.dtype, b: torch.dtype) -> torch.dtype:
    return torch.float32 if torch.float32 in (a, b) else a


class LayerNormAutoGrad(torch.autograd.Function):
    """
    Autodiff for layer normalisation; same call contract as the reference's
    ``LayerNormAutoGrad.apply(input, weight, bias, eps, autocast_to_fp32)``.  One more optional
    argument, ``output_dtype``, stores the output in that dtype instead of the one the rule above
    gives; ``LayerNormLinear`` passes the operand dtype of its projection.
    """
    @staticmethod
    def forward(ctx, input: Tensor, weight: Optional[Tensor] = None, bias: Optional[Tensor] = None,
                eps: float = 1e-5, autocast_to_fp32: bool = True,
                output_dtype: Optional[torch.dtype] = None) -> Tensor:
        _require_cuda(input, 'input')
        flattened_input = input.unsqueeze(0) if input.ndim == 1 else input
        flattened_input = flattened_input.flatten(0, -2)
        if flattened_input.stride(-1) != 1 or (flattened_input.shape[0] > 1 and
                                               flattened_input.stride(0) < flattened_input.shape[1]):
            flattened_input = flattened_input.contiguous()
        batch_dim, feat_dim = flattened_input.shape

        if output_dtype is None:
            output_dtype = get_norm_dtype(input.dtype, autocast_to_fp32)
        scale_by_weight = weight is not None
        add_bias = scale_by_weight and bias is not None
        requires_grad = (input.requires_grad or
                         (scale_by_weight and weight.requires_grad) or
                         (add_bias and bias.requires_grad))
        weight_op = bias_op = None
        if scale_by_weight:
            _require_cuda(weight, 'weight')
            weight_op = weight if weight.is_contiguous() else weight.contiguous()
            if add_bias:
                bias_op = bias if (bias.is_contiguous() and bias.dtype is weight.dtype) \
                    else bias.to(weight.dtype).contiguous()

        lib = _lib.load()
        with torch.cuda.device(input.device):
            stream = torch.cuda.current_stream().cuda_stream
            output = torch.empty((batch_dim, feat_dim), dtype=output_dtype, device=input.device)
            mean = inv_std = None
            if requires_grad:
                stats = torch.empty((2, batch_dim), dtype=torch.float32, device=input.device)
                mean, inv_std = stats[0], stats[1]
            _lib.check(lib.ab200_layer_norm_forward(
                _ptr(flattened_input), _ptr(weight_op), _ptr(bias_op), _ptr(mean), _ptr(inv_std), _ptr(output),
                batch_dim, feat_dim, flattened_input.stride(0) if batch_dim > 1 else feat_dim, feat_dim,
                _dtype_id(input.dtype), _dtype_id(weight_op.dtype) if scale_by_weight else 0,
                _dtype_id(output_dtype), float(eps), stream), 'ab200_layer_norm_forward')

        ctx.scale_by_weight = scale_by_weight
        ctx.add_bias = add_bias
        ctx.output_dtype = output_dtype
        ctx.input_shape = input.shape
        if requires_grad:
            ctx.save_for_backward(flattened_input, mean, inv_std, weight_op)
        return output.view(input.shape)

    @staticmethod
    def backward(ctx, output_grad: Tensor) -> Tuple[Optional[Tensor], ...]:
        flattened_input, mean, inv_std, weight = ctx.saved_tensors
        batch_dim, feat_dim = flattened_input.shape
        grad = output_grad.reshape(batch_dim, feat_dim)
        if grad.dtype is not ctx.output_dtype:
            grad = grad.to(ctx.output_dtype)
        if grad.stride(-1) != 1 or (batch_dim > 1 and grad.stride(0) < feat_dim):
            grad = grad.contiguous()          # e.g. the expanded gradient of y.sum()
        # The reference stores the input gradient in the forward's output dtype and leaves the cast to
        # the input's dtype to the autograd engine (attorch/layer_norm_layer.py:117-118); a narrower
        # output than input (the fused projection operand) keeps the input's dtype instead.
        grad_dtype = _wider(flattened_input.dtype, ctx.output_dtype)
        lib = _lib.load()
        with torch.cuda.device(flattened_input.device):
            device = flattened_input.device
            stream = torch.cuda.current_stream().cuda_stream
            input_grad = torch.empty((batch_dim, feat_dim), dtype=grad_dtype, device=device)
            weight_grad = bias_grad = workspace = None
            ws_bytes = 0
            if ctx.scale_by_weight:
                param_grads = torch.empty((2 if ctx.add_bias else 1, feat_dim), dtype=torch.float32, device=device)
                weight_grad = param_grads[0]
                bias_grad = param_grads[1] if ctx.add_bias else None
                ws_bytes = int(lib.ab200_layer_norm_workspace_bytes(batch_dim, feat_dim))
                workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
            _lib.check(lib.ab200_layer_norm_backward(
                _ptr(grad), _ptr(flattened_input), _ptr(mean), _ptr(inv_std), _ptr(weight), _ptr(input_grad),
                _ptr(weight_grad), _ptr(bias_grad), batch_dim, feat_dim,
                grad.stride(0) if batch_dim > 1 else feat_dim,
                flattened_input.stride(0) if batch_dim > 1 else feat_dim, feat_dim,
                _dtype_id(grad.dtype), _dtype_id(flattened_input.dtype),
                _dtype_id(weight.dtype) if weight is not None else 0, _dtype_id(grad_dtype),
                _ptr(workspace), ws_bytes, _ptr(_stream_scratch(device)['status']), stream),
                'ab200_layer_norm_backward')
        # One slot per forward argument (attorch/layer_norm_layer.py:151-153 pads with None).
        return input_grad.view(ctx.input_shape), weight_grad, bias_grad, None, None, None


class LayerNorm(nn.LayerNorm):
    """
    Layer-normalizes the input.  Same constructor as the reference's ``attorch.LayerNorm``
    (attorch/layer_norm_layer.py:156-213), including ``autocast_to_fp32``: PyTorch autocasts the output
    of layer normalisation to fp32; with the flag off the input dtype flows through.

    Args:
        normalized_shape: Dimensionality of last feature that is normalized.
        eps: Epsilon added in the square root in the denominator to avoid division by zero.
        elementwise_affine: Flag for scaling the normalized output by weights.
        bias: Flag for adding a bias vector to the normalized output if elementwise_affine is True.
        autocast_to_fp32: Flag for autocasting the output dtype to fp32.
            If False, the input dtype flows through.
        device: Device to use.
        dtype: Dtype of layer.

    Raises:
        RuntimeError: Normalized shape was not an integer.
    """
    def __init__(self, normalized_shape: int, eps: float = 1e-5, elementwise_affine: bool = True,
                 bias: bool = True, autocast_to_fp32: bool = True, device='cuda',
                 dtype: torch.dtype = torch.float32) -> None:
        if not isinstance(normalized_shape, int):
            raise RuntimeError('Normalized shape must be an integer.')
        super().__init__(normalized_shape, eps, elementwise_affine, bias, device, dtype)
        self.autocast_to_fp32 = autocast_to_fp32

    def forward(self, input: Tensor, output_dtype: Optional[torch.dtype] = None) -> Tensor:
        return LayerNormAutoGrad.apply(input, self.weight, self.bias, self.eps, self.autocast_to_fp32,
                                       output_dtype)


class LayerNormLinear(nn.Module):
    """
    ``linear(norm(input))`` for a ``LayerNorm`` and the ``Linear`` that follows it, as in a transformer
    block's ``self.mlp(self.ln2(output))`` (examples/wikitext-2/gpt.py:82, 30-37).  Under autocast the
    normalisation stores its output directly in the projection's operand dtype, so the fp32 output of
    the normalisation and the projection's cast pass over it (2.5 full passes over the activations)
    never exist; backward hands the projection's input gradient to the normalisation in that dtype too.
    The values are those of the two layers run one after the other: the operand the projection would
    make by casting the fp32 output is that output rounded once, which is what the fused store writes,
    and the input gradient the projection computes in the autocast dtype is widened either way.
    Without autocast (one dtype throughout) there is nothing to fuse and the two layers simply run.

    Args:
        norm: The normalisation layer.
        linear: The projection (with its own fused activation, bias, ...).
    """
    def __init__(self, norm: LayerNorm, linear: Linear) -> None:
        super().__init__()
        self.norm = norm
        self.linear = linear

    def forward(self, input: Tensor) -> Tensor:
        operand_dtype = linear_output_dtype(input.dtype)
        natural = get_norm_dtype(input.dtype, self.norm.autocast_to_fp32)
        fuse = operand_dtype is not natural and input.dtype in (torch.float32, operand_dtype)
        return self.linear(self.norm(input, operand_dtype if fuse else None))
