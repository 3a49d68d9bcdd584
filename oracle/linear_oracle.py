"""
TEST INFRASTRUCTURE - CPU oracle for the fused linear layer.  Not part of the product: only
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import it.

A plain torch-on-CPU restatement of what the reference's ``attorch.Linear`` computes
(forward and backward), following its data flow and rounding points step by step:

    forward    attorch/linear_kernels.py:143-188  (fp32 accumulate, operand cast 161-163, bias cast
               171-172, pre-activation store 176-181, activation on the unrounded accumulator 183)
    dtype rule attorch/utils.py:27-60, attorch/linear_layer.py:80
    backward   attorch/linear_layer.py:125-161  (dZ in the pre-activation's dtype 137-139,
               matmuls in the output dtype 152-155, bias gradient as a sum over dZ 156)
    math       attorch/act_kernels.py:14-628     (formulas and piecewise conventions),
               655-721 / 759-832                 (which activations are evaluated in fp32 and which
               in the dtype of the loaded tensor)

Parity pinned: tests/test_oracle.py checks this file against golden vectors produced by the
reference itself (its Triton kernels run by the Triton CPU interpreter; generator
tests/golden/make_golden.py) for fp32 and fp16, all 22 activation settings, the piecewise
switch points, strided 3-D inputs, and the smallest configuration (fp32, 64 x 128 -> 256, bias, relu).  bf16 has no reference-made vectors
(the interpreter's bf16 dot product is broken); the bf16 rules are the fp16 rules with the
other 16-bit type, and on GPU boxes that have the reference the GPU tests compare against it.
"""

from typing import Optional, Tuple

import torch
from torch import Tensor

SELU_SCALE = 1.0507009873554805
SELU_ALPHA = 1.6732632423543772

# Activations whose dispatcher branch up-casts the argument to fp32 first
# (attorch/act_kernels.py:655-721 forward, 759-832 backward); the rest run in the loaded dtype.
FP32_ACTS = frozenset({'sigmoid', 'logsigmoid', 'tanh', 'gelu', 'geluapprox', 'silu', 'selu', 'mish',
                       'softplus', 'tanhshrink', 'elu', 'celu'})

ALL_ACT_FUNCS = [None, 'sigmoid', 'logsigmoid', 'tanh', 'relu', 'gelu', 'geluapprox', 'silu', 'relu6',
                 'hardsigmoid', 'hardtanh', 'hardswish', 'selu', 'mish', 'softplus', 'softsign',
                 'tanhshrink', 'leaky_relu_0.01', 'elu_1', 'celu_1', 'hardshrink_0.5',
                 'softshrink_0.5']


def parse_act_func(act_func: Optional[str]) -> Tuple[Optional[str], Optional[float]]:
    """Name / parameter split of attorch/linear_layer.py:65-69."""
    param = None
    if act_func is not None and '_' in act_func:
        comps = act_func.split('_')
        act_func = '_'.join(comps[:-1])
        param = float(comps[-1])
    return act_func, param


def _sigmoid(x: Tensor) -> Tensor:
    return 1 / (1 + torch.exp(-x))                                   # act_kernels.py:14-24


def _tanh(x: Tensor) -> Tensor:
    return 2 * _sigmoid(2 * x) - 1                                   # act_kernels.py:71-81


def act_forward(name: Optional[str], x: Tensor, param: Optional[float] = None) -> Tensor:
    """act(x), formulas of attorch/act_kernels.py:14-613; x is used in the dtype it comes in."""
    if name is None:
        return x
    zero = torch.zeros((), dtype=x.dtype)
    if name == 'sigmoid':
        return _sigmoid(x)
    if name == 'logsigmoid':
        return torch.log(_sigmoid(x))                                # 43-53
    if name == 'tanh':
        return _tanh(x)
    if name == 'relu':
        return torch.maximum(zero, x)                                # 100-110
    if name == 'gelu':
        return 0.5 * (1 + torch.erf(0.707106781 * x)) * x            # 128-139
    if name == 'geluapprox':
        return 0.5 * (1 + _tanh(0.7978845608 * x * (1 + 0.044715 * x * x))) * x   # 159-170
    if name == 'silu':
        return x * _sigmoid(x)                                       # 190-200
    if name == 'relu6':
        return torch.clamp(x, 0, 6)                                  # 219-229
    if name == 'hardsigmoid':
        return torch.clamp(x / 6 + 0.5, 0, 1)                        # 247-257
    if name == 'hardtanh':
        return torch.clamp(x, -1, 1)                                 # 275-285
    if name == 'hardswish':
        return x * torch.clamp(x + 3, 0, 6) / 6                      # 303-313
    if name == 'selu':
        return SELU_SCALE * (torch.maximum(zero, x) +
                             torch.minimum(zero, SELU_ALPHA * (torch.exp(x) - 1)))   # 331-344
    if name == 'mish':
        return x * _tanh(torch.log(1 + torch.exp(x)))                # 364-374
    if name == 'softplus':
        return torch.log(1 + torch.exp(x))                           # 395-405
    if name == 'softsign':
        return x / (1 + torch.abs(x))                                # 423-433
    if name == 'tanhshrink':
        return x - _tanh(x)                                          # 452-462
    if name == 'leaky_relu':
        return torch.maximum(zero, x) + param * torch.minimum(zero, x)   # 480-491
    if name == 'elu':
        return torch.where(x <= 0, param * (torch.exp(x) - 1), x)    # 510-521
    if name == 'celu':
        return torch.maximum(zero, x) + torch.minimum(zero, param * (torch.exp(x / param) - 1))  # 540-551
    if name == 'hardshrink':
        return torch.where(torch.abs(x) <= param, zero, x)           # 571-582
    if name == 'softshrink':
        return torch.where(x > param, x - param,
                           torch.where(x < -param, x + param, zero))  # 601-613
    raise ValueError(f'unknown activation {name!r}')


def act_grad(name: Optional[str], x: Tensor, param: Optional[float] = None) -> Tensor:
    """d act(x) / dx, formulas of attorch/act_kernels.py:28-628 (the *_grad functions)."""
    one = torch.ones((), dtype=x.dtype)
    zero = torch.zeros((), dtype=x.dtype)
    if name is None:
        return torch.ones_like(x)
    if name == 'sigmoid':
        s = _sigmoid(x)
        return s * (1 - s)                                           # 28-39
    if name == 'logsigmoid':
        return 1 / (1 + torch.exp(x))                                # 57-67
    if name == 'tanh':
        t = _tanh(x)
        return 1 - t * t                                             # 85-96
    if name == 'relu':
        return torch.where(x <= 0, zero, one)                        # 114-124
    if name == 'gelu':
        cdf = 0.5 * (1 + torch.erf(0.707106781 * x))
        return 0.39894228 * torch.exp(-0.5 * x * x) * x + cdf        # 143-155
    if name == 'geluapprox':
        t = _tanh(0.7978845608 * x * (1 + 0.044715 * x * x))
        return 0.5 * (1 + t + x * (1 - t * t) * 0.7978845608 * (1 + 3 * 0.044715 * x * x))   # 174-186
    if name == 'silu':
        s = _sigmoid(x)
        return s * (x * (1 - s) + 1)                                 # 204-215
    if name == 'relu6':
        return torch.where((0 < x) & (x < 6), one, zero)             # 233-243
    if name == 'hardsigmoid':
        return torch.where((-3 < x) & (x < 3), one / 6, zero)        # 261-271
    if name == 'hardtanh':
        return torch.where((-1 < x) & (x < 1), one, zero)            # 289-299
    if name == 'hardswish':
        return torch.where(x < -3, zero, torch.where(x <= 3, x / 3 + 0.5, one))   # 317-327
    if name == 'selu':
        return SELU_SCALE * torch.where(x <= 0, SELU_ALPHA * torch.exp(x), one)   # 348-360
    if name == 'mish':
        e = torch.exp(x)
        delta = e * (e + 2) + 2
        return e * (e * ((4 * x + 6) + e * (e + 4)) + 4 * (x + 1)) / (delta * delta)   # 378-391
    if name == 'softplus':
        return _sigmoid(x)                                           # 409-419
    if name == 'softsign':
        d = 1 + torch.abs(x)
        return 1 / (d * d)                                           # 437-448
    if name == 'tanhshrink':
        t = _tanh(x)
        return 1 - (1 - t * t)                                       # 466-476
    if name == 'leaky_relu':
        return torch.where(x <= 0, param * one, one)                 # 495-506
    if name == 'elu':
        return torch.where(x <= 0, param * torch.exp(x), one)        # 525-536
    if name == 'celu':
        return torch.where(x <= 0, torch.exp(x / param), one)        # 555-566
    if name == 'hardshrink':
        return torch.where(torch.abs(x) <= param, zero, one)         # 586-597
    if name == 'softshrink':
        return torch.where(torch.abs(x) <= param, zero, one)         # 617-628
    raise ValueError(f'unknown activation {name!r}')


def output_dtype_rule(input_dtype: torch.dtype, autocast_dtype: Optional[torch.dtype]) -> torch.dtype:
    """
    attorch/utils.py:27-60 as Linear uses it (autocast='fp16', attorch/linear_layer.py:80).
    ``autocast_dtype`` is None when autocast is off.  The reference asserts on bf16 autocast
    (attorch/utils.py:45); this restatement extends the rule the obvious way (bf16 autocast ->
    bf16 output), which is what the CUDA path implements.
    """
    if autocast_dtype is None or autocast_dtype is torch.float32:
        return input_dtype
    return autocast_dtype


def tf32_round(x: Tensor, mode: str = 'nearest') -> Tensor:
    """
    fp32 -> TF32 (10-bit mantissa), the precision a tensor core keeps of an fp32 operand when a dot
    product is allowed to use TF32 (attorch/linear_kernels.py:57,165).  ``mode='truncate'`` drops the
    low 13 bits, which is what the B200 tensor cores do with fp32 operands (pinned by
    tests/test_linear_gpu.py::test_tf32_operands_are_truncated); ``'nearest'`` rounds.
    """
    bits = x.contiguous().view(torch.int32)
    if mode == 'truncate':
        rounded = bits & ~0x1FFF
    elif mode == 'nearest':
        rounded = (bits + 0x1000) & ~0x1FFF
    else:
        raise ValueError(mode)
    return rounded.view(torch.float32)


def linear_forward(x: Tensor, weight: Tensor, bias: Optional[Tensor], act_func: Optional[str],
                   autocast_dtype: Optional[torch.dtype] = None, save_pre_act: bool = True,
                   tf32: Optional[str] = None) -> Tuple[Tensor, Optional[Tensor]]:
    """
    Returns (output, pre_act) exactly as attorch/linear_kernels.py:143-188 produces them:
    operands (cast to fp16 / the 16-bit output dtype if the output is 16-bit) are multiplied with
    fp32 accumulation (here: float64 accumulation of the exact products, rounded once to fp32);
    the bias (cast likewise) is added to the fp32 accumulator; the pre-activation is that value
    rounded to the output dtype; the activation is evaluated on the *unrounded* fp32 value and then
    rounded.  ``weight`` is ``[in_features, out_features]``.  ``tf32`` ('truncate' or 'nearest')
    reduces fp32 operands to TF32 first, as a GPU's tensor cores do; None keeps exact fp32 products,
    as the reference's CPU interpreter run does.
    """
    name, param = parse_act_func(act_func)
    out_dtype = output_dtype_rule(x.dtype, autocast_dtype)
    x2 = x.flatten(0, -2)
    w = weight
    b = bias
    if out_dtype in (torch.float16, torch.bfloat16):
        x2, w = x2.to(out_dtype), w.to(out_dtype)
        b = None if b is None else b.to(out_dtype)
    elif tf32 is not None:
        x2, w = tf32_round(x2.float(), tf32), tf32_round(w.float(), tf32)
    accum = (x2.double() @ w.double()).float()
    if b is not None:
        accum = accum + b.float()[None, :]
    pre_act = accum.to(out_dtype) if (save_pre_act and name is not None) else None
    out = act_forward(name, accum, param).to(out_dtype)
    return out.view(*x.shape[:-1], weight.shape[1]), pre_act


def linear_backward(output_grad: Tensor, x: Tensor, pre_act: Optional[Tensor], weight: Tensor,
                    act_func: Optional[str], out_dtype: torch.dtype,
                    bias: Optional[Tensor] = None, tf32: Optional[str] = None,
                    derivative_in_fp32: bool = False, round_to_out_dtype: bool = True,
                    derivative_rounded: bool = False, stored_derivative: Optional[Tensor] = None
                    ) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
    """
    Returns (dX, dW, db) following attorch/linear_layer.py:125-161.

    dZ = dY * act'(Z) is computed from the stored (rounded) pre-activation, in fp32 for the
    activations of FP32_ACTS and in Z's dtype otherwise, and stored in Z's dtype (137-148).  The
    two products run in ``out_dtype`` (the reference wraps them in torch.autocast(dtype=output
    dtype), 152-155; with fp32 that is a plain fp32 matmul): operands rounded to ``out_dtype``,
    fp32 accumulation, result rounded to ``out_dtype``.  db = dZ.sum(0) in dZ's dtype (156).  As
    the autograd engine does afterwards, each gradient is finally cast to the dtype of the tensor
    it belongs to.

    Three switches describe where the CUDA path deliberately differs from the reference, so that
    tests can compare like with like: ``tf32`` multiplies fp32 operands as TF32 (the reference's
    backward uses true fp32 products, its forward TF32); ``derivative_in_fp32`` evaluates every
    activation derivative in fp32 instead of Z's 16-bit dtype; ``round_to_out_dtype=False`` skips
    the intermediate rounding of dX / dW to the output dtype when the destination is wider (the
    CUDA kernels write the fp32 accumulator straight into fp32 gradients under autocast);
    ``derivative_rounded`` rounds act'(Z) to Z's dtype before it multiplies dY (the CUDA forward can
    save the derivative in place of Z); ``stored_derivative`` supplies that saved act'(Z) itself, so
    that backward is checked through the tensor it actually reads.
    """
    name, param = parse_act_func(act_func)
    dy = output_grad.flatten(0, -2)
    x2 = x.flatten(0, -2)
    if name is None:
        dz = dy
    elif stored_derivative is not None:
        # Stored in dY's dtype: the saved derivative itself may be kept in another 2-byte type (fp16 for
        # a bf16 layer), the product is rounded to the layer's own.
        dz = (dy.float() * stored_derivative.flatten(0, -2).float()).to(dy.dtype)
    else:
        z = pre_act.float() if (name in FP32_ACTS or derivative_in_fp32) else pre_act
        grad = act_grad(name, z, param)
        if derivative_rounded:
            grad = grad.to(pre_act.dtype).float()
        dz = (dy * grad).to(pre_act.dtype)

    def mm(a: Tensor, b: Tensor) -> Tensor:
        a, b = a.to(out_dtype), b.to(out_dtype)
        if tf32 is not None and out_dtype is torch.float32:
            a, b = tf32_round(a, tf32), tf32_round(b, tf32)
        product = (a.double() @ b.double()).float()
        return product.to(out_dtype) if round_to_out_dtype else product

    dx = mm(dz, weight.T).view_as(x).to(x.dtype)
    dw = mm(x2.T, dz).to(weight.dtype)
    db = None
    if bias is not None:
        db = dz.float().sum(dim=0).to(dz.dtype).to(bias.dtype)
    return dx, dw, db


def linear_forward_backward(x: Tensor, weight: Tensor, bias: Optional[Tensor], act_func: Optional[str],
                            output_grad: Tensor, autocast_dtype: Optional[torch.dtype] = None,
                            tf32: Optional[str] = None):
    """Convenience: (output, pre_act, dX, dW, db) of one training step of the layer."""
    out_dtype = output_dtype_rule(x.dtype, autocast_dtype)
    out, pre_act = linear_forward(x, weight, bias, act_func, autocast_dtype, tf32=tf32)
    dx, dw, db = linear_backward(output_grad.to(out_dtype), x, pre_act, weight, act_func, out_dtype, bias,
                                 tf32=tf32)
    return out, pre_act, dx, dw, db


# ------------------------------------------------------------------------------------------------
# Standalone activation layers with fused dropout (attorch/act_layers.py:20-117,
# attorch/act_kernels.py:840-927, attorch/dropout_kernels.py:12-46)
# ------------------------------------------------------------------------------------------------
def philox4x32_10(counter: 'np.ndarray', seed: int) -> 'np.ndarray':
    """
    Philox 4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011)
    for counters (c, 0, 0, 0) with c a uint64 array split into two 32-bit words, key (seed, 0).
    Returns an array [..., 4] of uint32.  Triton's tl.rand, from which the reference draws its
    dropout mask (attorch/dropout_kernels.py:26), is built on the same generator (triton 3.x,
    triton/language/random.py: philox, randint, uint_to_uniform_float).
    """
    import numpy as np
    c = np.asarray(counter, dtype=np.uint64)
    c0 = (c & np.uint64(0xFFFFFFFF)).astype(np.uint64)
    c1 = (c >> np.uint64(32)).astype(np.uint64)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = np.uint64(seed & 0xFFFFFFFF), np.uint64(0)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        n0 = ((p1 >> np.uint64(32)) ^ c1 ^ k0) & mask
        n1 = p1 & mask
        n2 = ((p0 >> np.uint64(32)) ^ c3 ^ k1) & mask
        n3 = p0 & mask
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint32)


def dropout_uniform(seed: int, n: int, stream: str = 'reference') -> Tensor:
    """
    The n uniform numbers in [0, 1) that decide the dropout mask of elements 0 .. n-1.

    'reference': tl.rand(seed, offset) as the reference calls it (attorch/dropout_kernels.py:26 with
    the int32 offsets of attorch/act_kernels.py:869-870): one Philox block per element, counter
    (offset, 0, 0, 0); its first word as int32, mirrored onto the non-negative half
    (w < 0 ? -w - 1 : w), converted to fp32 and scaled by 4.6566127342e-10.
    'packed': the CUDA library's cheaper stream: block index // 4, word index % 4, top 24 bits.
    """
    import numpy as np
    if stream == 'packed':
        blocks = philox4x32_10(np.arange((n + 3) // 4, dtype=np.uint64), seed).reshape(-1)[:n]
        return torch.from_numpy(((blocks >> np.uint32(8)).astype(np.float32) / np.float32(16777216.0)))
    if stream != 'reference':
        raise ValueError(stream)
    words = philox4x32_10(np.arange(n, dtype=np.uint64) & np.uint64(0xFFFFFFFF), seed)[..., 0]
    signed = words.astype(np.int64)
    signed = np.where(signed >= 2 ** 31, signed - 2 ** 32, signed)
    mirrored = np.where(signed < 0, -signed - 1, signed)
    return torch.from_numpy(mirrored.astype(np.float32) * np.float32(4.6566127342e-10))


def act_layer_forward(x: Tensor, act_func: str, drop_p: float = 0.0, seed: int = 0,
                      stream: str = 'reference') -> Tensor:
    """
    act_func_forward_kernel (attorch/act_kernels.py:840-880): the activation (in fp32 for the
    activations of FP32_ACTS, else in x's dtype), then apply_dropout
    (attorch/dropout_kernels.py:12-28): 0 where the uniform number is below drop_p, otherwise
    divided by 1 - drop_p; stored in x's dtype.
    """
    name, param = parse_act_func(act_func)
    z = x.float() if name in FP32_ACTS else x
    y = act_forward(name, z, param)
    if drop_p > 0:
        u = dropout_uniform(seed, x.numel(), stream).view(x.shape)
        y = torch.where(u < drop_p, torch.zeros((), dtype=y.dtype), y / (1 - drop_p))
    return y.to(x.dtype)


def act_layer_backward(dy: Tensor, x: Tensor, act_func: str, drop_p: float = 0.0, seed: int = 0,
                       stream: str = 'reference') -> Tensor:
    """
    act_func_backward_kernel (attorch/act_kernels.py:883-927): apply_dropout_grad
    (attorch/dropout_kernels.py:31-46) on dy, times act'(x); stored in x's dtype.
    """
    name, param = parse_act_func(act_func)
    z = x.float() if name in FP32_ACTS else x
    g = dy
    if drop_p > 0:
        u = dropout_uniform(seed, x.numel(), stream).view(x.shape)
        g = torch.where(u < drop_p, torch.zeros((), dtype=dy.dtype), dy / (1 - drop_p))
    return (g * act_grad(name, z, param)).to(x.dtype)


def glu_forward(x: Tensor, dim: int, act_func: str) -> Tensor:
    """
    glu_forward_kernel (attorch/glu_kernels.py:13-53) on the halves attorch/glu_layer.py:58-60 makes:
    x1 * act(x2), the activation in fp32 for the activations of FP32_ACTS, else in x's dtype; stored
    in x's dtype.
    """
    name, param = parse_act_func(act_func)
    x1, x2 = x.chunk(2, dim=dim)
    z = x2.float() if name in FP32_ACTS else x2
    return (x1 * act_forward(name, z, param)).to(x.dtype)


def glu_backward(dy: Tensor, x: Tensor, dim: int, act_func: str) -> Tensor:
    """
    glu_backward_kernel (attorch/glu_kernels.py:56-105): dx1 = dy * act(x2), dx2 = dy * x1 * act'(x2),
    concatenated along dim (attorch/glu_layer.py:116).
    """
    name, param = parse_act_func(act_func)
    x1, x2 = x.chunk(2, dim=dim)
    z = x2.float() if name in FP32_ACTS else x2
    g1 = (dy * act_forward(name, z, param)).to(x.dtype)
    g2 = (dy * x1 * act_grad(name, z, param)).to(x.dtype)
    return torch.cat([g1, g2], dim=dim)


def cross_entropy_forward(x: Tensor, target: Tensor, weight: Optional[Tensor] = None,
                          autocast: bool = False) -> Tensor:
    """
    cross_entropy_loss_forward_kernel (attorch/cross_entropy_loss_kernels.py:56-88) and the host code
    after it (attorch/cross_entropy_loss_layer.py:75-79): logits widened to fp32 (line 74), per row
    log(sum(exp(x - max))) - x[target] + max, times the target's class weight if weights are given;
    summed and divided by the batch size, or by the sum of the targets' weights.  Stored in fp32 under
    autocast, else in the logits' dtype (get_output_dtype(..., autocast='fp32'), line 58).
    """
    xf = x.float()
    mx = xf.max(dim=1).values
    rows = torch.arange(len(x))
    loss = torch.log(torch.exp(xf - mx[:, None]).sum(dim=1)) - xf[rows, target] + mx
    if weight is not None:
        w = weight.float()[target]
        total = (loss * w).sum() / w.sum()
    else:
        total = (loss / len(x)).sum() if len(x) else loss.sum()
    return total.to(torch.float32 if autocast else x.dtype)


def cross_entropy_backward(output_grad: Tensor, x: Tensor, target: Tensor, weight: Optional[Tensor] = None,
                           autocast: bool = False) -> Tensor:
    """
    cross_entropy_loss_backward_kernel (attorch/cross_entropy_loss_kernels.py:145-173):
    dL * (softmax(x) - onehot(target)), times weight[target] / sum of the targets' weights, or divided
    by the batch size; fp32 arithmetic, stored in the loss's dtype.
    """
    xf = x.float()
    softmax = torch.softmax(xf, dim=1)
    onehot = torch.zeros_like(xf)
    onehot[torch.arange(len(x)), target] = 1.0
    grad = output_grad.float() * (softmax - onehot)
    if weight is not None:
        w = weight.float()[target]
        grad = grad * (w / w.sum())[:, None]
    else:
        grad = grad / len(x)
    return grad.to(torch.float32 if autocast else x.dtype)


def layer_norm_forward(x: Tensor, weight: Optional[Tensor] = None, bias: Optional[Tensor] = None,
                       eps: float = 1e-5, output_dtype: Optional[torch.dtype] = None
                       ) -> Tuple[Tensor, Tensor, Tensor]:
    """
    layer_norm_forward_kernel (attorch/layer_norm_kernels.py:82-103): the row widened to fp32 (line 84),
    mean = sum / feat_dim, diff = x - mean, inv_std = rsqrt(sum(diff^2) / feat_dim + eps), output =
    diff * inv_std, then * weight, then + bias (bias only together with weight, attorch/
    layer_norm_layer.py:59-60), rounded once by the store.  A 1-D input is one row (attorch/
    layer_norm_layer.py:51).  Returns (output in output_dtype - the input's dtype unless given -,
    mean fp32, inv_std fp32).
    """
    rows = x.unsqueeze(0) if x.ndim == 1 else x
    rows = rows.flatten(0, -2).float()
    feat_dim = rows.shape[1]
    mean = rows.sum(dim=1) / feat_dim
    diff = rows - mean[:, None]
    inv_std = torch.rsqrt((diff * diff).sum(dim=1) / feat_dim + eps)
    out = diff * inv_std[:, None]
    if weight is not None:
        out = out * weight.float()
        if bias is not None:
            out = out + bias.float()
    return out.to(output_dtype or x.dtype).view(x.shape), mean, inv_std


def layer_norm_backward(output_grad: Tensor, x: Tensor, mean: Tensor, inv_std: Tensor,
                        weight: Optional[Tensor] = None, has_bias: bool = False,
                        grad_dtype: Optional[torch.dtype] = None
                        ) -> Tuple[Tensor, Optional[Tensor], Optional[Tensor]]:
    """
    layer_norm_backward_kernel (attorch/layer_norm_kernels.py:183-221) and the sums after it (attorch/
    layer_norm_layer.py:146-149): with pre_lin = (x - mean) * inv_std and g = weight * dy (dy without
    weights), dx = inv_std * (g - (pre_lin * sum(pre_lin * g) / feat_dim + sum(g) / feat_dim));
    weight_grad = sum over rows of dy * pre_lin, bias_grad = sum over rows of dy, both fp32.  dx is
    stored in the forward's output dtype (attorch/layer_norm_layer.py:117-118).
    """
    rows = (x.unsqueeze(0) if x.ndim == 1 else x).flatten(0, -2).float()
    dy = output_grad.reshape(rows.shape).float()
    feat_dim = rows.shape[1]
    pre_lin = (rows - mean[:, None]) * inv_std[:, None]
    g = weight.float() * dy if weight is not None else dy
    term1 = pre_lin * ((pre_lin * g).sum(dim=1) / feat_dim)[:, None]
    term2 = (g.sum(dim=1) / feat_dim)[:, None]
    dx = inv_std[:, None] * (g - (term1 + term2))
    weight_grad = (dy * pre_lin).sum(dim=0) if weight is not None else None
    bias_grad = dy.sum(dim=0) if (weight is not None and has_bias) else None
    return dx.to(grad_dtype or output_grad.dtype).view(x.shape), weight_grad, bias_grad
