"""
A projection followed by a gated linear unit, ``GLU(act_func)(Linear(in, 2 * out)(x))``, as one layer
whose forward pass is one kernel: the GEMM's epilogue holds both halves of a row block of the
projection in tensor memory, stores them (backward needs them) and writes ``x1 * act(x2)`` next to
them, instead of a second pass that reads the ``[tokens, 2 * out]`` pre-activation back
(``ab200_gated_linear_forward``).  The reference composes the two layers (attorch/linear_layer.py:164-205,
attorch/glu_layer.py:119-138, e.g. the gated up-projection of a transformer MLP); results are those of
that composition bit for bit, because the halves are multiplied as they are stored.

Parameters have the layout of ``attorch_b200.Linear(in_features, 2 * out_features)``: ``weight``
``[in_features, 2 * out_features]`` (first half of the columns: the values, second half: the gate),
``bias`` ``[2 * out_features]``.  Backward is the composition's: the gated unit's backward kernel on the
stored halves, the bias sum, and the two products of the linear layer.
"""

from typing import Optional, Tuple

import torch
from torch import Tensor, nn

from . import _lib
from .acts import act_id, parse_act_func
from .linear_layer import (_as_operand, _cached_size, _dtype_id, _flags_for, _ptr, _require_cuda, _stream_scratch,
                           _workspace, get_output_dtype)


class GatedLinearAutoGrad(torch.autograd.Function):
    """``apply(input, weight, bias, act_func)`` -> ``x1 * act(x2)`` with ``[x1 | x2] = input @ weight + bias``."""
    @staticmethod
    def forward(ctx, input: Tensor, weight: Tensor, bias: Optional[Tensor], act_func: str) -> Tensor:
        assert weight.ndim == 2 and weight.shape[1] % 2 == 0, \
            f'Weights must be 2D with an even number of columns, received shape {weight.shape}'
        assert input.shape[-1] == weight.shape[0], \
            f'Incompatible input ({input.shape}) and weights ({weight.shape}) shape'
        assert bias is None or (bias.ndim == 1 and bias.shape[0] == weight.shape[1]), \
            f'Incompatible weights ({weight.shape}) and bias shape'
        name, param = parse_act_func(act_func)
        _require_cuda(input, 'input')
        _require_cuda(weight, 'weight')
        flat = input.flatten(0, -2)
        rows, in_dim = flat.shape
        half = weight.shape[1] // 2
        out_dtype = get_output_dtype(input.dtype)
        lib = _lib.load()
        with torch.cuda.device(input.device):
            stream = torch.cuda.current_stream().cuda_stream
            status = _ptr(_stream_scratch(input.device)['status'])
            x_op = _as_operand(flat, out_dtype, stream)
            w_op = _as_operand(weight, out_dtype, stream)
            bias_op = bias if (bias is None or bias.is_contiguous()) else bias.contiguous()
            pre_act = torch.empty((rows, 2 * half), dtype=out_dtype, device=input.device)
            output = torch.empty((rows, half), dtype=out_dtype, device=input.device)
            dt = _dtype_id(out_dtype)
            rc = lib.ab200_gated_linear_forward(
                _ptr(x_op), _ptr(w_op), _ptr(bias_op), _ptr(pre_act), _ptr(output), rows, in_dim, half,
                x_op.stride(0), x_op.stride(1), w_op.stride(0), w_op.stride(1), 2 * half, half, dt, dt,
                _dtype_id(bias_op.dtype) if bias_op is not None else 0, act_id(name), 0.0 if param is None else param,
                status, stream, _flags_for(input.device))
            ctx.fused = rc == 0
            if rc == -5:
                # Operands the tensor-core kernel cannot address: the two kernels of the composition.
                ws_bytes = _cached_size('ab200_forward_workspace_bytes', rows, in_dim, 2 * half, 0)
                workspace = _workspace(input.device, ws_bytes) if ws_bytes else None
                _lib.check(lib.ab200_linear_forward(
                    _ptr(x_op), _ptr(w_op), _ptr(bias_op), None, _ptr(pre_act), rows, in_dim, 2 * half,
                    x_op.stride(0), x_op.stride(1), w_op.stride(0), w_op.stride(1), 2 * half, 2 * half, dt, dt,
                    _dtype_id(bias_op.dtype) if bias_op is not None else 0, 0, 0.0, _ptr(workspace), ws_bytes,
                    status, stream, _flags_for(input.device)), 'ab200_linear_forward')
                _lib.check(lib.ab200_glu_forward(_ptr(pre_act), _ptr(output), rows, half, dt, act_id(name),
                                                 0.0 if param is None else param, stream), 'ab200_glu_forward')
            else:
                _lib.check(rc, 'ab200_gated_linear_forward')
        ctx.act, ctx.param = act_id(name), 0.0 if param is None else param
        ctx.input_shape, ctx.input_dtype = input.shape, input.dtype
        ctx.weight_dtype, ctx.bias_dtype = weight.dtype, None if bias is None else bias.dtype
        ctx.needs = (input.requires_grad, weight.requires_grad, bias is not None and bias.requires_grad)
        ctx.out_dtype = out_dtype
        if any(ctx.needs):
            ctx.save_for_backward(x_op, w_op, pre_act)
        return output.view(*input.shape[:-1], half)

    @staticmethod
    def backward(ctx, output_grad: Tensor) -> Tuple[Optional[Tensor], ...]:
        x_op, w_op, pre_act = ctx.saved_tensors
        rows, in_dim = x_op.shape
        half = pre_act.shape[1] // 2
        lib = _lib.load()
        device = x_op.device
        dt = _dtype_id(ctx.out_dtype)
        input_grad = weight_grad = bias_grad = None
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream().cuda_stream
            status = _ptr(_stream_scratch(device)['status'])
            dy = output_grad.reshape(rows, half).to(ctx.out_dtype).contiguous()
            # dZ = [dy * act(x2) | dy * x1 * act'(x2)]  (attorch/glu_kernels.py:56-105)
            dz = torch.empty_like(pre_act)
            _lib.check(lib.ab200_glu_backward(_ptr(dy), _ptr(pre_act), _ptr(dz), rows, half, dt, ctx.act, ctx.param,
                                              stream), 'ab200_glu_backward')
            if ctx.needs[2]:
                bias_grad = torch.empty(2 * half, dtype=ctx.bias_dtype, device=device)
                ws_bytes = _cached_size('ab200_act_backward_workspace_bytes', rows, 2 * half)
                workspace = _workspace(device, ws_bytes)
                _lib.check(lib.ab200_act_backward(_ptr(dz), None, None, _ptr(bias_grad), rows, 2 * half, 2 * half,
                                                  2 * half, 2 * half, dt, _dtype_id(bias_grad.dtype), 0, 0.0,
                                                  _ptr(workspace), ws_bytes, stream), 'ab200_act_backward')
            if ctx.needs[1]:
                weight_grad = torch.empty((in_dim, 2 * half), dtype=ctx.weight_dtype, device=device)
                ws_bytes = _cached_size('ab200_gemm_workspace_bytes', in_dim, 2 * half, rows)
                workspace = _workspace(device, ws_bytes) if ws_bytes else None
                _lib.check(lib.ab200_linear_backward_weight(
                    _ptr(x_op), _ptr(dz), _ptr(weight_grad), rows, in_dim, 2 * half, x_op.stride(0), x_op.stride(1),
                    2 * half, 1, 2 * half, dt, _dtype_id(weight_grad.dtype), _ptr(workspace), ws_bytes, status, stream,
                    _flags_for(device)), 'ab200_linear_backward_weight')
            if ctx.needs[0]:
                input_grad = torch.empty((rows, in_dim), dtype=ctx.input_dtype, device=device)
                ws_bytes = _cached_size('ab200_gemm_workspace_bytes', rows, in_dim, 2 * half)
                workspace = _workspace(device, ws_bytes) if ws_bytes else None
                _lib.check(lib.ab200_linear_backward_input(
                    _ptr(dz), _ptr(w_op), _ptr(input_grad), rows, in_dim, 2 * half, 2 * half, 1, w_op.stride(0),
                    w_op.stride(1), in_dim, dt, _dtype_id(input_grad.dtype), _ptr(workspace), ws_bytes, status, stream,
                    _flags_for(device)), 'ab200_linear_backward_input')
                input_grad = input_grad.view(ctx.input_shape)
        return input_grad, weight_grad, bias_grad, None


class GatedLinear(nn.Module):
    """
    ``GLU(dim=-1, act_func)(Linear(in_features, 2 * out_features, bias)(input))`` with the gated unit fused
    into the projection's epilogue.

    Args:
        in_features: Number of input features.
        out_features: Number of output features (the projection has twice as many columns).
        bias: Flag for additive bias.
        act_func: Activation applied to the gate half; same options as ``Linear`` (default ``'sigmoid'``,
            as ``attorch.GLU``).
        device: Device to use.
        dtype: Dtype of layer.
    """
    def __init__(self, in_features: int, out_features: int, bias: bool = True, act_func: str = 'sigmoid',
                 device='cuda', dtype: torch.dtype = torch.float32) -> None:
        super().__init__()
        from .linear_layer import Linear
        projection = Linear(in_features, 2 * out_features, bias=bias, device=device, dtype=dtype)
        self.in_features, self.out_features, self.act_func = in_features, out_features, act_func
        self.weight = projection.weight
        self.bias = projection.bias

    def forward(self, input: Tensor) -> Tensor:
        return GatedLinearAutoGrad.apply(input, self.weight, self.bias, self.act_func)

    def extra_repr(self) -> str:
        return (f'in_features={self.in_features}, out_features={self.out_features}, '
                f'bias={self.bias is not None}, act_func={self.act_func!r}')
