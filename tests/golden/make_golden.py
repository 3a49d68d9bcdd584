"""
Generates the golden vectors under tests/golden/ by running the REFERENCE implementation
(BobMcDear/attorch, its own Triton kernels executed by Triton's CPU interpreter) on seeded inputs.

Usage (needs a checkout of the reference; no GPU):

    python tests/golden/make_golden.py --reference /path/to/attorch-checkout

The reference is imported unmodified.  Two host-side shims make it importable without a GPU:
``torch.cuda.get_device_capability`` is stubbed (the reference queries it at import time,
attorch/utils.py:12-24), and each autotuner is cut down to its first configuration so that no
config is benchmarked (attorch/linear_kernels.py:44-56, attorch/act_kernels.py:840-887,
attorch/glu_kernels.py:13-16 and 56-59).

Each case is stored as one .npz with the inputs (or the seed that regenerates them plus a
checksum) and the reference's output, dX, dW and db; the standalone activation layers go into
act_layers_fp32.npz, the gated linear unit into glu_fp32.npz, bf16 runs of both (element-wise
kernels only) into elementwise_bf16.npz, the cross-entropy loss into cross_entropy_fp32.npz, layer
normalisation into layer_norm.npz and, in bf16, layer_norm_bf16.npz.  The linear layer itself is not generated in bf16: the
interpreter's bf16 dot product returns garbage.
"""

import argparse
import hashlib
import os
import sys
from pathlib import Path

os.environ['TRITON_INTERPRET'] = '1'

import numpy as np
import torch

OUT_DIR = Path(__file__).resolve().parent

ALL_ACT_FUNCS = [None, 'sigmoid', 'logsigmoid', 'tanh', 'relu', 'gelu', 'geluapprox', 'silu', 'relu6',
                 'hardsigmoid', 'hardtanh', 'hardswish', 'selu', 'mish', 'softplus', 'softsign',
                 'tanhshrink', 'leaky_relu_0.01', 'elu_1', 'celu_1', 'hardshrink_0.5',
                 'softshrink_0.5']


def load_reference(path: str):
    torch.cuda.get_device_capability = lambda *args, **kwargs: (10, 0)
    sys.path.insert(0, path)
    import attorch
    from attorch.act_kernels import act_func_backward_kernel, act_func_forward_kernel
    from attorch.glu_kernels import glu_backward_kernel, glu_forward_kernel
    from attorch.linear_kernels import linear_forward_kernel
    linear_forward_kernel.configs = linear_forward_kernel.configs[:1]
    act_func_backward_kernel.configs = act_func_backward_kernel.configs[:1]
    act_func_forward_kernel.configs = act_func_forward_kernel.configs[:1]
    glu_forward_kernel.configs = glu_forward_kernel.configs[:1]
    glu_backward_kernel.configs = glu_backward_kernel.configs[:1]
    return attorch


def checksum(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def run_reference(attorch, x, weight, bias, act_func, dy):
    """One forward + backward of the reference layer with the given parameter values."""
    layer = attorch.Linear(weight.shape[0], weight.shape[1], bias=bias is not None,
                           act_func=act_func, device='cpu', dtype=weight.dtype)
    with torch.no_grad():
        layer.weight.copy_(weight)
        if bias is not None:
            layer.bias.copy_(bias)
    x = x.clone().requires_grad_(True)
    y = layer(x)
    y.backward(dy)
    return (y.detach(), x.grad, layer.weight.grad,
            layer.bias.grad if bias is not None else None)


def to_np(t):
    if t is None:
        return np.zeros(0, dtype=np.float32)
    return t.detach().float().numpy() if t.dtype is torch.bfloat16 else t.detach().numpy()


def save(name, store_inputs, x, w, b, dy, outs, **meta):
    y, dx, dw, db = outs
    data = dict(y=to_np(y), dx=to_np(dx), dw=to_np(dw), db=to_np(db),
                input_checksum=np.array(checksum(to_np(x), to_np(w), to_np(b), to_np(dy))))
    if store_inputs:
        data.update(x=to_np(x), w=to_np(w), b=to_np(b), dy=to_np(dy))
    for key, value in meta.items():
        data[key] = np.array(value)
    np.savez_compressed(OUT_DIR / f'{name}.npz', **data)
    print(f'wrote {name}.npz')


def config1_inputs():
    """The smallest configuration: fp32, X [64, 128], 128 -> 256, bias, relu, every draw under seed 0."""
    torch.manual_seed(0)
    x = torch.randn(64, 128)
    torch.manual_seed(0)
    linear = torch.nn.Linear(128, 256, bias=True)
    w = linear.weight.detach().T.contiguous()
    b = linear.bias.detach().clone()
    torch.manual_seed(0)
    dy = torch.randn(64, 256)
    return x, w, b, dy


def small_inputs(seed, dtype, shape=(3, 5, 35), out_dim=50, strided=True):
    """A strided 3-D input (every other row of a taller tensor), K = 35, N = 50."""
    gen = torch.Generator().manual_seed(seed)
    if strided:
        tall = torch.randn((shape[0], 2 * shape[1], shape[2]), generator=gen).to(dtype)
        x = tall[:, ::2, :]
    else:
        x = torch.randn(shape, generator=gen).to(dtype)
    w = (torch.randn((shape[-1], out_dim), generator=gen) / shape[-1] ** 0.5).to(dtype)
    b = torch.randn(out_dim, generator=gen).to(dtype)
    dy = torch.randn((*shape[:-1], out_dim), generator=gen).to(dtype)
    return x, w, b, dy


def switch_point_inputs():
    """
    Pre-activations that hit the piecewise switch points exactly (the points the reference's
    tests/test_act_layers.py:55-82 checks): W is the identity and the bias zero, so Z == X.
    """
    points = torch.tensor([-6.0, -3.0, -1.0, -0.5, 0.0, 0.5, 1.0, 3.0, 6.0, 7.0, -7.0, 2.0,
                           -2.0, 0.25, -0.25, 5.0])
    x = points.repeat(4, 1)                      # [4, 16]
    w = torch.eye(16)
    b = torch.zeros(16)
    dy = torch.arange(1, 65, dtype=torch.float32).view(4, 16) / 8
    return x, w, b, dy


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument('--reference', required=True, help='path of a checkout of BobMcDear/attorch')
    args = parser.parse_args()
    attorch = load_reference(args.reference)

    x, w, b, dy = config1_inputs()
    save('config1_fp32_relu', False, x, w, b, dy, run_reference(attorch, x, w, b, 'relu', dy),
         act_func='relu', dtype='float32')

    for act_func in ALL_ACT_FUNCS:
        tag = 'none' if act_func is None else act_func.replace('.', 'p')
        x, w, b, dy = small_inputs(1, torch.float32)
        save(f'small_fp32_{tag}', True, x, w, b, dy, run_reference(attorch, x, w, b, act_func, dy),
             act_func=str(act_func), dtype='float32')
        x, w, b, dy = switch_point_inputs()
        save(f'switch_fp32_{tag}', True, x, w, b, dy, run_reference(attorch, x, w, b, act_func, dy),
             act_func=str(act_func), dtype='float32')

    for act_func in [None, 'relu', 'gelu', 'silu', 'hardswish', 'softsign', 'leaky_relu_0.01', 'mish']:
        tag = 'none' if act_func is None else act_func.replace('.', 'p')
        x, w, b, dy = small_inputs(2, torch.float16, shape=(4, 6, 40), out_dim=48)
        save(f'small_fp16_{tag}', True, x, w, b, dy, run_reference(attorch, x, w, b, act_func, dy),
             act_func=str(act_func), dtype='float16')

    # No bias, 2-D input.
    x, w, _, dy = small_inputs(3, torch.float32, shape=(7, 24), out_dim=40, strided=False)
    save('small_fp32_nobias_gelu', True, x, w, None, dy, run_reference(attorch, x, w, None, 'gelu', dy),
         act_func='gelu', dtype='float32')

    act_layer_goldens(attorch)
    glu_goldens(attorch)
    elementwise_bf16_goldens(attorch)
    cross_entropy_goldens(attorch)
    layer_norm_goldens(attorch)
    layer_norm_bf16_goldens(attorch)


ACT_LAYERS = [('Sigmoid', {}), ('LogSigmoid', {}), ('Tanh', {}), ('ReLU', {}), ('GELU', {}),
              ('GELU', {'approximate': 'tanh'}), ('SiLU', {}), ('ReLU6', {}), ('Hardsigmoid', {}),
              ('Hardtanh', {}), ('Hardswish', {}), ('SELU', {}), ('Mish', {}), ('Softplus', {}),
              ('Softsign', {}), ('Tanhshrink', {}), ('LeakyReLU', {'negative_slope': 0.01}),
              ('ELU', {'alpha': 1.0}), ('CELU', {'alpha': 1.0}), ('Hardshrink', {'lambd': 0.5}),
              ('Softshrink', {'lambd': 0.5})]


def act_layer_goldens(attorch):
    """
    The reference's standalone activation layers (attorch/act_layers.py): for every layer class the
    output and input gradient on a seeded input that also contains the piecewise switch points, without
    dropout and with drop_p = 0.5 and 0.3.  The layer draws its dropout seed with random.randint(0, 65535)
    (attorch/act_layers.py:54); Python's generator is seeded just before, and the seed the layer drew is
    stored beside the result, so that the vectors pin WHICH elements are dropped for a given seed.
    """
    import random
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(6, 40, generator=gen) * 2
    x[0, :12] = torch.tensor([-6.0, -3.0, -1.0, -0.5, 0.0, 0.5, 1.0, 3.0, 6.0, 7.0, -7.0, 2.0])
    dy = torch.randn(6, 40, generator=gen)
    data = {'x': x.numpy(), 'dy': dy.numpy()}
    for index, (name, kwargs) in enumerate(ACT_LAYERS):
        for drop_p, label in ((0.0, 'plain'), (0.5, 'drop'), (0.3, 'drop30')):
            layer = getattr(attorch, name)(drop_p=drop_p, **kwargs)
            layer.train()
            xin = x.clone().requires_grad_(True)
            random.seed(1000 + 3 * index + len(label))
            drawn = random.randint(0, 65535)
            random.seed(1000 + 3 * index + len(label))
            y = layer(xin)
            y.backward(dy)
            tag = f'{index:02d}_{name}_{label}'
            data[f'y_{tag}'] = y.detach().numpy()
            data[f'dx_{tag}'] = xin.grad.numpy()
            data[f'seed_{tag}'] = np.array(drawn)
    np.savez_compressed(OUT_DIR / 'act_layers_fp32.npz', **data)
    print('wrote act_layers_fp32.npz')


GLU_CASES = [((6, 10), -1), ((6, 10), 0), ((4, 6, 5), 1), ((2, 3, 8), 2), ((2, 4, 3, 2), -3)]


def glu_goldens(attorch):
    """
    The reference's gated linear unit (attorch/glu_layer.py) for every activation setting on a 2-D
    input gated over its last dimension, and for sigmoid / gelu / relu over every dimension of inputs
    with 2 to 4 dimensions: output and input gradient.
    """
    gen = torch.Generator().manual_seed(5)
    data = {}
    for case, (shape, dim) in enumerate(GLU_CASES):
        x = torch.randn(shape, generator=gen) * 2
        out_shape = list(shape)
        out_shape[dim] //= 2
        dy = torch.randn(out_shape, generator=gen)
        data[f'x_{case}'] = x.numpy()
        data[f'dy_{case}'] = dy.numpy()
        acts = [a for a in ALL_ACT_FUNCS if a is not None] if case == 0 else ['sigmoid', 'gelu', 'relu']
        for act_func in acts:
            xin = x.clone().requires_grad_(True)
            y = attorch.GLU(dim=dim, act_func=act_func)(xin)
            y.backward(dy)
            tag = f'{case}_{act_func.replace(".", "p")}'
            data[f'y_{tag}'] = y.detach().numpy()
            data[f'dx_{tag}'] = xin.grad.numpy()
    np.savez_compressed(OUT_DIR / 'glu_fp32.npz', **data)
    print('wrote glu_fp32.npz')


def elementwise_bf16_goldens(attorch):
    """
    bf16 vectors of the reference's element-wise kernels (the interpreter's bf16 dot product is broken,
    its element-wise arithmetic is not): every standalone activation layer - whose backward is the
    act_func_backward_kernel the linear layer's backward launches too (attorch/linear_layer.py:143-146) -
    and the gated linear unit, on bf16 inputs that contain the piecewise switch points.  These pin
    the arithmetic in front of the final store.  Two properties of the interpreter limit what they pin:
    it converts fp32 to bf16 by dropping the low 16 bits (a GPU rounds to nearest even), and it gets
    products of two bf16 tensors wrong (the second half of every GLU gradient and everything hardshrink
    touches in the GLU come out with magnitudes of 1e30; the tests leave those entries alone).  Values
    are saved as fp32 arrays holding bf16 numbers.
    """
    gen = torch.Generator().manual_seed(6)
    x = (torch.randn(6, 40, generator=gen) * 2).bfloat16()
    x[0, :12] = torch.tensor([-6.0, -3.0, -1.0, -0.5, 0.0, 0.5, 1.0, 3.0, 6.0, 7.0, -7.0, 2.0]).bfloat16()
    dy = torch.randn(6, 40, generator=gen).bfloat16()
    data = {'x': x.float().numpy(), 'dy': dy.float().numpy()}
    skipped = []
    for index, (name, kwargs) in enumerate(ACT_LAYERS):
        layer = getattr(attorch, name)(**kwargs)
        xin = x.clone().requires_grad_(True)
        try:
            y = layer(xin)
            y.backward(dy)
        except Exception as error:   # triton 3.6: the interpreter cannot make the bf16 constants some kernels use
            if 'get_bf16' not in repr(error):
                raise
            skipped.append(f'{index:02d}_{name}')
            continue
        assert y.dtype is torch.bfloat16
        data[f'y_{index:02d}_{name}'] = y.detach().float().numpy()
        data[f'dx_{index:02d}_{name}'] = xin.grad.float().numpy()
    gx = (torch.randn(6, 10, generator=gen) * 2).bfloat16()
    gdy = torch.randn(6, 5, generator=gen).bfloat16()
    data['glu_x'], data['glu_dy'] = gx.float().numpy(), gdy.float().numpy()
    for act_func in [a for a in ALL_ACT_FUNCS if a is not None]:
        xin = gx.clone().requires_grad_(True)
        tag = act_func.replace('.', 'p')
        try:
            y = attorch.GLU(dim=-1, act_func=act_func)(xin)
            y.backward(gdy)
        except Exception as error:
            if 'get_bf16' not in repr(error):
                raise
            skipped.append(f'glu_{tag}')
            continue
        assert y.dtype is torch.bfloat16
        data[f'glu_y_{tag}'] = y.detach().float().numpy()
        data[f'glu_dx_{tag}'] = xin.grad.float().numpy()
    data['skipped'] = np.array(','.join(skipped))
    np.savez_compressed(OUT_DIR / 'elementwise_bf16.npz', **data)
    print('wrote elementwise_bf16.npz; the interpreter could not run:', skipped)


CROSS_ENTROPY_CASES = [(1, 8, False), (16, 10, False), (16, 10, True), (37, 50, True), (5, 1000, False),
                       (64, 257, True)]


def cross_entropy_goldens(attorch):
    """
    The reference's cross-entropy loss (attorch/cross_entropy_loss_layer.py) in fp32: logits scaled so
    that rows have a wide range, targets drawn uniformly, with and without class weights; the loss and
    the gradient of the logits for an upstream gradient of 1 (loss.backward()) and of 0.5.
    """
    from attorch.cross_entropy_loss_kernels import cross_entropy_loss_backward_kernel, \
        cross_entropy_loss_forward_kernel
    cross_entropy_loss_forward_kernel.configs = cross_entropy_loss_forward_kernel.configs[:1]
    cross_entropy_loss_backward_kernel.configs = cross_entropy_loss_backward_kernel.configs[:1]
    gen = torch.Generator().manual_seed(8)
    data = {}
    for case, (batch, classes, weighted) in enumerate(CROSS_ENTROPY_CASES):
        x = torch.randn(batch, classes, generator=gen) * 3
        target = torch.randint(0, classes, (batch,), generator=gen)
        weight = torch.rand(classes, generator=gen) + 0.1 if weighted else None
        data[f'x_{case}'], data[f'target_{case}'] = x.numpy(), target.numpy()
        if weighted:
            data[f'weight_{case}'] = weight.numpy()
        for scale, label in ((1.0, 'unit'), (0.5, 'half')):
            xin = x.clone().requires_grad_(True)
            loss = attorch.CrossEntropyLoss(weight=weight)(xin, target)
            (loss * scale).backward()
            data[f'loss_{case}'] = loss.detach().numpy()
            data[f'dx_{case}_{label}'] = xin.grad.numpy()
    np.savez_compressed(OUT_DIR / 'cross_entropy_fp32.npz', **data)
    print('wrote cross_entropy_fp32.npz')


LAYER_NORM_CASES = [
    # shape, dtype, elementwise_affine, bias, eps
    ((16,), 'float32', True, True, 1e-5),
    ((5, 40), 'float32', True, True, 1e-5),
    ((5, 40), 'float32', True, False, 1e-6),
    ((5, 40), 'float32', False, False, 1e-5),
    ((3, 7, 96), 'float32', True, True, 1e-5),
    ((2049, 2), 'float32', True, True, 1e-5),        # several rows per program in the reference, ragged
    ((257, 33), 'float32', True, True, 1e-5),
    ((6, 1100), 'float32', True, True, 1e-5),
    ((4, 6, 64), 'float16', True, True, 1e-5),
    ((9, 200), 'float16', True, False, 1e-5),
    ((9, 200), 'float16', False, False, 1e-6),
]


def layer_norm_goldens(attorch):
    """
    The reference's layer normalisation (attorch/layer_norm_layer.py) on fp32 and fp16 inputs: output,
    input gradient and, with an affine transform, the gradients of weight and bias, for a normal upstream
    gradient.  Weights and biases are drawn from N(0, 1) as the reference's own test does
    (tests/test_layer_norm_layer.py:40-49); inputs get an offset and a scale per row so that mean and
    variance differ between rows.
    """
    from attorch.layer_norm_kernels import layer_norm_backward_kernel, layer_norm_forward_kernel
    layer_norm_forward_kernel.configs = layer_norm_forward_kernel.configs[:1]
    layer_norm_backward_kernel.configs = layer_norm_backward_kernel.configs[:1]
    gen = torch.Generator().manual_seed(9)
    data = {}
    for case, (shape, dtype_name, affine, bias, eps) in enumerate(LAYER_NORM_CASES):
        dtype = getattr(torch, dtype_name)
        rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
        x = torch.randn(shape, generator=gen)
        if len(shape) > 1:
            scale = (torch.rand(rows, generator=gen) * 3 + 0.2).view(*shape[:-1], 1)
            shift = (torch.randn(rows, generator=gen) * 2).view(*shape[:-1], 1)
            x = x * scale + shift
        x = x.to(dtype)
        dy = torch.randn(shape, generator=gen).to(dtype)
        layer = attorch.LayerNorm(shape[-1], eps, affine, bias, device='cpu', dtype=dtype)
        if affine:
            with torch.no_grad():
                layer.weight.copy_(torch.randn(shape[-1], generator=gen))
                if bias:
                    layer.bias.copy_(torch.randn(shape[-1], generator=gen))
        xin = x.clone().requires_grad_(True)
        y = layer(xin)
        y.backward(dy)
        assert y.dtype is dtype and xin.grad.dtype is dtype
        data[f'x_{case}'], data[f'dy_{case}'] = to_np(x), to_np(dy)
        data[f'y_{case}'], data[f'dx_{case}'] = to_np(y), to_np(xin.grad)
        if affine:
            data[f'w_{case}'], data[f'dw_{case}'] = to_np(layer.weight), to_np(layer.weight.grad)
            if bias:
                data[f'b_{case}'], data[f'db_{case}'] = to_np(layer.bias), to_np(layer.bias.grad)
    np.savez_compressed(OUT_DIR / 'layer_norm.npz', **data)
    print('wrote layer_norm.npz')


LAYER_NORM_BF16_CASES = [
    # shape, parameter dtype, bias
    ((7, 40), 'bfloat16', True),
    ((33, 200), 'bfloat16', False),
    ((4, 6, 64), 'float32', True),
    ((5, 1040), 'bfloat16', True),
]


def layer_norm_bf16_goldens(attorch):
    """
    bf16 runs of the reference's layer normalisation (its kernels have no dot product, so the interpreter
    runs them): bf16 inputs and upstream gradients, bf16 or fp32 parameters.  As with the other bf16 vectors,
    the interpreter stores fp32 results as bf16 by dropping the low 16 bits where a GPU rounds to nearest, so
    these pin the fp32 value in front of the store.  Values are saved as fp32 arrays holding bf16 numbers.
    """
    from attorch.layer_norm_kernels import layer_norm_backward_kernel, layer_norm_forward_kernel
    layer_norm_forward_kernel.configs = layer_norm_forward_kernel.configs[:1]
    layer_norm_backward_kernel.configs = layer_norm_backward_kernel.configs[:1]
    gen = torch.Generator().manual_seed(10)
    data = {}
    for case, (shape, param_dtype_name, bias) in enumerate(LAYER_NORM_BF16_CASES):
        param_dtype = getattr(torch, param_dtype_name)
        rows = int(np.prod(shape[:-1]))
        x = torch.randn(shape, generator=gen) * (torch.rand(rows, generator=gen) * 3 + 0.2).view(*shape[:-1], 1) \
            + (torch.randn(rows, generator=gen) * 2).view(*shape[:-1], 1)
        x = x.bfloat16()
        dy = torch.randn(shape, generator=gen).bfloat16()
        layer = attorch.LayerNorm(shape[-1], bias=bias, device='cpu', dtype=param_dtype)
        with torch.no_grad():
            layer.weight.copy_(torch.randn(shape[-1], generator=gen))
            if bias:
                layer.bias.copy_(torch.randn(shape[-1], generator=gen))
        xin = x.clone().requires_grad_(True)
        y = layer(xin)
        y.backward(dy)
        assert y.dtype is torch.bfloat16 and xin.grad.dtype is torch.bfloat16
        data[f'x_{case}'], data[f'dy_{case}'] = to_np(x), to_np(dy)
        data[f'y_{case}'], data[f'dx_{case}'] = to_np(y), to_np(xin.grad)
        data[f'w_{case}'], data[f'dw_{case}'] = to_np(layer.weight), to_np(layer.weight.grad)
        if bias:
            data[f'b_{case}'], data[f'db_{case}'] = to_np(layer.bias), to_np(layer.bias.grad)
    np.savez_compressed(OUT_DIR / 'layer_norm_bf16.npz', **data)
    print('wrote layer_norm_bf16.npz')


if __name__ == '__main__':
    main()
