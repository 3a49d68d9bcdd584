"""
Drop-in replacement for ``attorch.Linear`` (attorch/linear_layer.py:164-205 of the reference) whose
device work runs in hand-written sm_100a CUDA kernels behind a C ABI (include/attorch_b200.h).

``Y = act(X @ W + b)`` with ``W`` of shape ``[in_features, out_features]``; forward and backward
(``dX``, ``dW``, ``db``).  This module only mirrors the reference's host logic - argument checks,
activation-string parsing, flattening, the autocast / output-dtype rule, which tensors are saved
and which gradients are produced - and hands raw device pointers to the library.  There is no
Triton, no PyTorch matmul and no CPU path: on a machine without the built library or without a
CUDA device the layer raises.
"""

from typing import Dict, Optional, Tuple

import torch
from torch import Tensor, nn

from . import _lib
from .acts import act_id, parse_act_func

_DTYPE_IDS = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}

# Per (device index, stream) scratch: a grow-only workspace and the device status word.
_scratch: Dict[Tuple[int, int], Dict[str, Tensor]] = {}
_scratch_clock = 0

# Flags forwarded to every GEMM entry point (tests use them to pin a kernel family).
_gemm_flags = 0

# What forward keeps for backward when there is an activation: the pre-activation Z, as the
# reference does (attorch/linear_layer.py:104-105), or act'(Z) computed in the same epilogue.  The
# second makes the activation backward one multiply per element instead of a second evaluation of
# the activation's transcendental functions; it costs one extra rounding of the derivative to the
# 16-bit storage type.
_save_derivative = True


def set_save_derivative(enabled: bool) -> bool:
    """Chooses what forward saves for backward (see above); returns the previous setting."""
    global _save_derivative
    previous, _save_derivative = _save_derivative, bool(enabled)
    return previous


# Per device index: SMs the persistent GEMM kernels leave free (for a collective that runs beside
# them); handed to every GEMM call in bits 16-23 of its flags.
_reserved_sms: Dict[int, int] = {}


def set_reserved_sms(device_index: int, sms: int) -> int:
    """
    Makes every GEMM launched on that device from now on leave ``sms`` SMs free (0: none);
    returns the previous value.  A data-parallel step sets it while its gradient exchange is in
    flight: a persistent GEMM that held every SM would make the collective wait for it to end.
    """
    previous = _reserved_sms.get(device_index, 0)
    _reserved_sms[device_index] = max(0, min(255, int(sms)))
    return previous


def _flags_for(device: torch.device) -> int:
    reserve = _reserved_sms.get(device.index, 0) if _reserved_sms else 0
    return _gemm_flags | (reserve << _lib.FLAG_RESERVE_SMS_SHIFT)


def set_gemm_flags(flags: int) -> int:
    """Sets the AB200_FLAG_* bits passed to the GEMM entry points; returns the previous value."""
    global _gemm_flags
    previous, _gemm_flags = _gemm_flags, int(flags)
    return previous


def get_output_dtype(input_dtype: torch.dtype) -> torch.dtype:
    """
    Output dtype of the layer: the CUDA autocast dtype while autocast is enabled, else the input
    dtype.  The reference (attorch/utils.py:27-60 with autocast='fp16', attorch/linear_layer.py:80)
    returns fp16 under autocast and asserts that the autocast dtype is fp16 or fp32; here bf16
    autocast is accepted too and yields bf16, and fp32 "autocast" leaves the input dtype alone.
    """
    if torch.is_autocast_enabled('cuda'):
        dtype = torch.get_autocast_dtype('cuda')
        assert dtype in (torch.float32, torch.float16, torch.bfloat16), \
            'Only fp16, bf16 and fp32 casting are supported'
        return input_dtype if dtype is torch.float32 else dtype
    return input_dtype


def _dtype_id(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_IDS[dtype]
    except KeyError:
        raise TypeError(f'Unsupported dtype {dtype}; supported: float32, float16, bfloat16') from None


def _ptr(tensor: Optional[Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _stream_scratch(device: torch.device) -> Dict[str, Tensor]:
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    global _scratch_clock
    entry = _scratch.get(key)
    if entry is None:
        entry = {'status': torch.zeros(1, dtype=torch.int32, device=device),
                 'workspace': torch.empty(0, dtype=torch.uint8, device=device)}
        _scratch[key] = entry
    _scratch_clock += 1
    entry['used'] = _scratch_clock
    return entry


_size_cache: Dict[Tuple, int] = {}


def _cached_size(func_name: str, *shape: int) -> int:
    """Workspace sizes depend on the shape only: ask the library once per shape."""
    key = (func_name,) + shape
    size = _size_cache.get(key)
    if size is None:
        size = int(getattr(_lib.load(), func_name)(*shape))
        _size_cache[key] = size
    return size


def _workspace(device: torch.device, nbytes: int) -> Tensor:
    entry = _stream_scratch(device)
    if entry['workspace'].numel() < nbytes:
        entry['workspace'] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return entry['workspace']


def check_status(device: Optional[torch.device] = None) -> None:
    """
    Synchronises and raises if any kernel launched through this module gave up on a bounded wait
    (the device status word of include/attorch_b200.h).  The layer never synchronises on its
    own; call this where the program synchronises anyway.
    """
    failure = None
    for key, entry in list(_scratch.items()):
        if device is not None and device.index is not None and device.index != key[0]:
            continue
        code = int(entry['status'].item())          # synchronises with the stream that last used the entry
        if code != 0 and failure is None:
            entry['status'].zero_()
            failure = code
    _trim_scratch()
    if failure is not None:
        raise _lib.LibraryError(f'device status {failure}: {_lib.error_string(failure)}')


_MAX_SCRATCH_ENTRIES = 32


def _trim_scratch() -> None:
    """
    Drops the scratch entries (status word, workspace) of streams that have not been used for longest once
    there are more than _MAX_SCRATCH_ENTRIES of them.  Called from check_status(), after every status word
    has been read, i.e. when no kernel that could still write one is in flight.
    """
    if len(_scratch) <= _MAX_SCRATCH_ENTRIES:
        return
    by_age = sorted(_scratch.items(), key=lambda item: item[1].get('used', 0))
    for key, _ in by_age[:len(_scratch) - _MAX_SCRATCH_ENTRIES]:
        del _scratch[key]


def _require_cuda(tensor: Tensor, what: str) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(
            f'attorch_b200.Linear runs only on CUDA devices (sm_100a); {what} is on {tensor.device}. '
            'There is no CPU fallback.')


def _tma_addressable(tensor: Tensor) -> bool:
    """Unit inner stride, 16-byte aligned base and row pitch."""
    elt = tensor.element_size()
    return (tensor.stride(1) == 1 and tensor.data_ptr() % 16 == 0
            and tensor.stride(0) >= tensor.shape[1] and (tensor.stride(0) * elt) % 16 == 0)


def _as_operand(tensor: Tensor, dtype: torch.dtype, stream: int) -> Tensor:
    """
    Returns a 2-D operand of ``dtype`` that the kernels can read: the tensor itself if it already
    has that dtype and TMA can address it (or a copy could not make it addressable either),
    otherwise a contiguous converted copy made by the library's cast kernel.
    """
    rows, cols = tensor.shape
    if tensor.dtype is dtype:
        copy_helps = (cols * tensor.element_size()) % 16 == 0
        if _tma_addressable(tensor) or not copy_helps:
            return tensor
    out = torch.empty((rows, cols), dtype=dtype, device=tensor.device)
    if out.numel():
        lib = _lib.load()
        _lib.check(lib.ab200_cast_2d(tensor.data_ptr(), out.data_ptr(), rows, cols,
                                     tensor.stride(0), tensor.stride(1),
                                     _dtype_id(tensor.dtype), _dtype_id(dtype), stream),
                   'ab200_cast_2d')
    return out


class LinearAutoGrad(torch.autograd.Function):
    """
    Autodiff for the fused linear layer; same call contract as the reference's
    ``LinearAutoGrad`` (attorch/linear_layer.py:19-161): ``apply(input, weight, bias, act_func)``.
    Three optional trailing arguments serve data-parallel training: the buffers ``dW`` and ``db``
    are written into (e.g. views of a flat all-reduce bucket), and a callable ``grad_ready(i, n)``
    that backward invokes each time block ``i`` of ``n`` row blocks of ``dW`` is enqueued (``db`` is
    complete before block 0), before ``dX`` is, so that the gradient exchange of this layer can
    overlap the remaining work; ``dw_chunks`` is ``n``.  ``defer_input_grad``, if given, is called with
    a function that launches the ``dX`` product instead of launching it: backward then returns the
    buffer ``dX`` will be written to once the caller runs that function (on any stream ordered after
    backward), which lets a data-parallel step start its gradient exchange before ``dX``.  ``residual``, a tensor
    of the output's shape, is added to the output after the activation inside the kernel's epilogue
    (``act(X W + b) + R``); its gradient is the upstream gradient.
    """
    @staticmethod
    def forward(ctx, input: Tensor, weight: Tensor, bias: Optional[Tensor] = None,
                act_func: Optional[str] = None, weight_grad_out: Optional[Tensor] = None,
                bias_grad_out: Optional[Tensor] = None, grad_ready=None, dw_chunks: int = 1,
                defer_input_grad=None, residual: Optional[Tensor] = None) -> Tensor:
        assert weight.ndim == 2, \
            f'Weights must be 2D, received shape {weight.shape}'
        assert bias is None or bias.ndim == 1, \
            f'Bias must be 1D, received shape {bias.shape}'
        assert input.shape[-1] == weight.shape[0], \
            f'Incompatible input ({input.shape}) and weights ({weight.shape}) shape'
        assert bias is None or weight.shape[1] == bias.shape[0], \
            f'Incompatible weights ({weight.shape}) and bias ({bias.shape}) shape'

        name, param = parse_act_func(act_func)
        _require_cuda(input, 'input')
        _require_cuda(weight, 'weight')

        flattened_input = input.flatten(0, -2)
        batch_dim, in_feat_dim = flattened_input.shape
        _, out_feat_dim = weight.shape

        requires_grad = (input.requires_grad or weight.requires_grad or
                         (bias is not None and bias.requires_grad) or
                         (residual is not None and residual.requires_grad))
        save_pre_act = requires_grad and (name is not None)

        output_dtype = get_output_dtype(input.dtype)
        op_dtype = output_dtype  # operands are multiplied in the output dtype (fp32 -> TF32)
        lib = _lib.load()

        with torch.cuda.device(input.device):
            stream = torch.cuda.current_stream().cuda_stream
            scratch = _stream_scratch(input.device)
            x_op = _as_operand(flattened_input, op_dtype, stream)
            w_op = _as_operand(weight, op_dtype, stream)
            # With a 16-bit output the reference rounds the bias to that dtype before adding it to
            # the fp32 accumulator (attorch/linear_kernels.py:171-172); the kernels do that themselves.
            bias_op = bias
            if bias_op is not None and not bias_op.is_contiguous():
                bias_op = bias_op.contiguous()

            saves_derivative = save_pre_act and _save_derivative
            output = torch.empty((batch_dim, out_feat_dim), device=input.device, dtype=output_dtype)
            # A bf16 layer keeps act'(Z) as fp16: same size, three more mantissa bits, so that
            # dZ = dY * act'(Z) is in effect rounded once, as the reference's dZ is.
            derivative_fp16 = saves_derivative and output_dtype is torch.bfloat16
            pre_act = (torch.empty((batch_dim, out_feat_dim), device=input.device,
                                   dtype=torch.float16 if derivative_fp16 else output_dtype)
                       if save_pre_act else None)

            ws_bytes = _cached_size('ab200_forward_workspace_bytes', batch_dim, in_feat_dim, out_feat_dim, _gemm_flags)
            workspace = _workspace(input.device, ws_bytes) if ws_bytes else None
            residual_op = None
            if residual is not None:
                assert residual.shape == (*input.shape[:-1], out_feat_dim), \
                    f'Incompatible residual ({residual.shape}) and output shape'
                _require_cuda(residual, 'residual')
                residual_op = residual.reshape(batch_dim, out_feat_dim)
                if residual_op.dtype is not output_dtype or residual_op.stride(1) != 1 or \
                        (batch_dim > 1 and residual_op.stride(0) < out_feat_dim):
                    # Another dtype or layout than the kernel reads: one strided, converting copy.
                    dense = torch.empty((batch_dim, out_feat_dim), dtype=output_dtype, device=input.device)
                    if dense.numel():
                        _lib.check(lib.ab200_cast_2d(
                            residual_op.data_ptr(), dense.data_ptr(), batch_dim, out_feat_dim,
                            residual_op.stride(0), residual_op.stride(1), _dtype_id(residual_op.dtype),
                            _dtype_id(output_dtype), stream), 'ab200_cast_2d')
                    residual_op = dense
            _lib.check(lib.ab200_linear_forward_residual(
                _ptr(x_op), _ptr(w_op), _ptr(bias_op), _ptr(pre_act), _ptr(output), _ptr(residual_op),
                batch_dim, in_feat_dim, out_feat_dim,
                x_op.stride(0), x_op.stride(1), w_op.stride(0), w_op.stride(1),
                out_feat_dim, out_feat_dim,
                residual_op.stride(0) if residual_op is not None and batch_dim > 1 else out_feat_dim,
                _dtype_id(op_dtype), _dtype_id(output_dtype),
                _dtype_id(bias_op.dtype) if bias_op is not None else 0,
                act_id(name), 0.0 if param is None else param,
                _ptr(workspace), ws_bytes, _ptr(scratch['status']), stream,
                _flags_for(input.device) | (_lib.FLAG_SAVE_DERIVATIVE if saves_derivative else 0) |
                (_lib.FLAG_DERIVATIVE_FP16 if derivative_fp16 else 0)),
                'ab200_linear_forward_residual')

        ctx.residual_requires_grad = residual is not None and residual.requires_grad
        ctx.residual_dtype = None if residual is None else residual.dtype
        ctx.param = param
        ctx.act_func = name
        ctx.bias_requires_grad = False if bias is None else bias.requires_grad
        ctx.bias_dtype = None if bias is None else bias.dtype
        ctx.output_dtype = output_dtype
        ctx.input_shape = input.shape
        ctx.input_dtype = input.dtype
        ctx.input_requires_grad = input.requires_grad
        ctx.weight_requires_grad = weight.requires_grad
        ctx.weight_dtype = weight.dtype
        ctx.weight_shape = weight.shape
        ctx.has_grad_out = (weight_grad_out is not None, bias_grad_out is not None)
        ctx.grad_ready = grad_ready
        ctx.dw_chunks = int(dw_chunks)
        ctx.defer_input_grad = defer_input_grad
        ctx.saved_derivative = requires_grad and name is not None and _save_derivative
        if requires_grad:
            # Backward multiplies in the output dtype, so the converted operands are what it
            # needs; keeping them avoids converting X and W a second time.
            saved = [x_op, pre_act, w_op]
            if weight_grad_out is not None:
                saved.append(weight_grad_out)
            if bias_grad_out is not None:
                saved.append(bias_grad_out)
            ctx.save_for_backward(*saved)

        return output.view(*input.shape[:-1], out_feat_dim)

    @staticmethod
    def backward(ctx, output_grad: Tensor) -> Tuple[Optional[Tensor], ...]:
        saved = list(ctx.saved_tensors)
        x_op, pre_act, w_op = saved[:3]
        extra = saved[3:]
        weight_grad_out = extra.pop(0) if ctx.has_grad_out[0] else None
        bias_grad_out = extra.pop(0) if ctx.has_grad_out[1] else None

        batch_dim, in_feat_dim = x_op.shape
        out_feat_dim = w_op.shape[1]
        op_dtype = ctx.output_dtype
        lib = _lib.load()
        device = x_op.device

        input_grad = weight_grad = bias_grad = None
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream().cuda_stream
            scratch = _stream_scratch(device)
            status = _ptr(scratch['status'])
            # The upstream gradient may arrive with any strides (expanded, transposed, ...).
            dy = _as_operand(output_grad.reshape(batch_dim, out_feat_dim), op_dtype, stream)
            if dy.stride(1) != 1 or dy.stride(0) < out_feat_dim:
                dy = dy.contiguous()

            need_db = ctx.bias_requires_grad
            if need_db:
                bias_grad = (bias_grad_out if bias_grad_out is not None else
                             torch.empty(out_feat_dim, dtype=ctx.bias_dtype, device=device))
            if ctx.act_func is None:
                pre_act_grad = dy
            else:
                pre_act_grad = torch.empty((batch_dim, out_feat_dim), dtype=op_dtype, device=device)
            if ctx.act_func is not None or need_db:
                ws_bytes = _cached_size('ab200_act_backward_workspace_bytes', batch_dim, out_feat_dim) if need_db else 0
                workspace = _workspace(device, ws_bytes) if ws_bytes else None
                _lib.check(lib.ab200_act_backward(
                    _ptr(dy), _ptr(pre_act),
                    _ptr(pre_act_grad) if ctx.act_func is not None else None,
                    _ptr(bias_grad) if need_db else None,
                    batch_dim, out_feat_dim, dy.stride(0),
                    pre_act.stride(0) if pre_act is not None else out_feat_dim,
                    pre_act_grad.stride(0), _dtype_id(op_dtype),
                    _dtype_id(bias_grad.dtype) if need_db else 0,
                    (_lib.ACT_SAVED_DERIVATIVE_F16 if pre_act.dtype is not op_dtype else _lib.ACT_SAVED_DERIVATIVE)
                    if ctx.saved_derivative else act_id(ctx.act_func),
                    0.0 if ctx.param is None else ctx.param,
                    _ptr(workspace), ws_bytes, stream), 'ab200_act_backward')

            # dW before dX: in a data-parallel step the all-reduce of dW can then start while
            # dX is still being computed.
            if ctx.weight_requires_grad:
                weight_grad = (weight_grad_out if weight_grad_out is not None else
                               torch.empty(ctx.weight_shape, dtype=ctx.weight_dtype, device=device))
                # dW is computed in `chunks` blocks of rows (= input features).  With a gradient
                # exchange attached, block i is handed to it as soon as it is enqueued, so that the
                # exchange of block i overlaps the computation of block i + 1 and of dX.
                chunks = ctx.dw_chunks if (ctx.grad_ready is not None and ctx.dw_chunks > 1 and
                                           in_feat_dim % (ctx.dw_chunks * 8) == 0) else 1
                rows = in_feat_dim // chunks
                ws_bytes = _cached_size('ab200_gemm_workspace_bytes', rows, out_feat_dim, batch_dim)
                workspace = _workspace(device, ws_bytes) if ws_bytes else None
                for c in range(chunks):
                    x_part = x_op[:, c * rows:(c + 1) * rows]
                    dw_part = weight_grad[c * rows:(c + 1) * rows]
                    _lib.check(lib.ab200_linear_backward_weight(
                        _ptr(x_part), _ptr(pre_act_grad), _ptr(dw_part),
                        batch_dim, rows, out_feat_dim,
                        x_part.stride(0), x_part.stride(1), pre_act_grad.stride(0), pre_act_grad.stride(1),
                        dw_part.stride(0), _dtype_id(op_dtype), _dtype_id(weight_grad.dtype),
                        _ptr(workspace), ws_bytes, status, stream, _flags_for(device)),
                        'ab200_linear_backward_weight')
                    if ctx.grad_ready is not None:
                        ctx.grad_ready(c, chunks)
            elif ctx.grad_ready is not None:
                ctx.grad_ready(0, 1)
            if ctx.input_requires_grad:
                input_grad = torch.empty((batch_dim, in_feat_dim), dtype=ctx.input_dtype, device=device)
                dx_ptr, dx_dtype = input_grad.data_ptr(), _dtype_id(input_grad.dtype)

                # Holds dZ and W alive but not dX: autograd must remain the only owner of the
                # tensor it is handed, or it would copy it before the deferred product has run.
                # Rows [row_begin, row_end) of dX; a data-parallel step may launch the product in two
                # pieces, the first beside its gradient exchange (on fewer SMs), the rest after it.
                dx_row_bytes = in_feat_dim * input_grad.element_size()

                def launch_input_grad(row_begin=0, row_end=None, dz=pre_act_grad, w=w_op):
                    row_end = batch_dim if row_end is None else min(row_end, batch_dim)
                    rows = row_end - row_begin
                    if rows <= 0:
                        return
                    with torch.cuda.device(device):
                        run_stream = torch.cuda.current_stream().cuda_stream
                        run_scratch = _stream_scratch(device)
                        nbytes = _cached_size('ab200_gemm_workspace_bytes', rows, in_feat_dim, out_feat_dim)
                        space = _workspace(device, nbytes) if nbytes else None
                        _lib.check(lib.ab200_linear_backward_input(
                            dz.data_ptr() + row_begin * dz.stride(0) * dz.element_size(), _ptr(w),
                            dx_ptr + row_begin * dx_row_bytes,
                            rows, in_feat_dim, out_feat_dim,
                            dz.stride(0), dz.stride(1), w.stride(0), w.stride(1),
                            in_feat_dim, _dtype_id(op_dtype), dx_dtype,
                            _ptr(space), nbytes, _ptr(run_scratch['status']), run_stream, _flags_for(device)),
                            'ab200_linear_backward_input')

                if ctx.defer_input_grad is not None:
                    ctx.defer_input_grad(launch_input_grad)
                else:
                    launch_input_grad()
                input_grad = input_grad.view(ctx.input_shape)

        # One slot per forward argument (attorch/linear_layer.py:158-161 pads with None).  A gradient
        # that was written into a caller-supplied buffer is not returned as well: autograd would
        # accumulate a copy of it into ``.grad`` (the buffer's owner, e.g. a gradient bucket, binds
        # ``.grad`` to the buffer itself).
        residual_grad = output_grad.to(ctx.residual_dtype) if ctx.residual_requires_grad else None
        if weight_grad_out is not None:
            weight_grad = None
        if bias_grad_out is not None:
            bias_grad = None
        return input_grad, weight_grad, bias_grad, None, None, None, None, None, None, residual_grad


class Linear(nn.Linear):
    """
    Linearly transforms the input using weights, optionally adding bias and fusing an activation
    function.  Same constructor, parameters and state_dict as the reference's ``attorch.Linear``
    (attorch/linear_layer.py:164-205).

    Note: as in the reference, the weight matrix is of shape ``[in_features, out_features]``,
    the transpose of ``torch.nn.Linear``'s.

    Args:
        in_features: Number of input features.
        out_features: Number of output features.
        bias: Flag for additive bias.
        act_func: Name of activation function to apply, with None for identity.
            Options are 'sigmoid', 'logsigmoid', 'tanh', 'relu', 'gelu', 'geluapprox', 'silu',
            'relu6', 'hardsigmoid', 'hardtanh', 'hardswish', 'selu', 'mish', 'softplus',
            'softsign', 'tanhshrink', 'leaky_relu_PARAM', 'elu_PARAM', 'celu_PARAM',
            'hardshrink_PARAM', and 'softshrink_PARAM' (e.g. 'leaky_relu_0.01').
        device: Device to use.
        dtype: Dtype of layer.
    """
    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 act_func: Optional[str] = None, device='cuda',
                 dtype: torch.dtype = torch.float32) -> None:
        super().__init__(in_features, out_features, bias, device, dtype)
        self.weight = nn.Parameter(self.weight.T.contiguous())
        self.act_func = act_func
        # Optional (dW, db) destination buffers, e.g. views into a gradient bucket.
        self.weight_grad_out: Optional[Tensor] = None
        self.bias_grad_out: Optional[Tensor] = None
        # Optional callable run in backward as blocks of dW are enqueued (see LinearAutoGrad).
        self.grad_ready = None
        self.dw_chunks = 1
        # Optional callable that receives the launcher of dX instead of dX being launched (see LinearAutoGrad).
        self.defer_input_grad = None

    def forward(self, input: Tensor, residual: Optional[Tensor] = None) -> Tensor:
        """
        ``act(input @ weight + bias)``, as the reference's layer; with ``residual`` (a tensor of the
        output's shape) the kernel's epilogue adds it to the result, which saves the separate pass
        a caller's ``x + linear(...)`` makes over the output.
        """
        return LinearAutoGrad.apply(input, self.weight, self.bias, self.act_func,
                                    self.weight_grad_out, self.bias_grad_out, self.grad_ready,
                                    self.dw_chunks, self.defer_input_grad, residual)
