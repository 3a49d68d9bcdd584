"""
GPU parity of the standalone activation layers with fused dropout (attorch_b200.act_layers, through
the C ABI) against the reference's golden vectors and the CPU oracle.
"""

import random

import pytest
import torch

import attorch_b200
from oracle import linear_oracle as oracle
from tests.helpers import ACT_LAYERS, load_act_layer_golden

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def run(layer, x, dy):
    xg = x.to(DEV).requires_grad_(True)
    y = layer(xg)
    y.backward(dy.to(DEV).to(y.dtype))
    return y.detach().cpu(), xg.grad.cpu()


@pytest.mark.parametrize('index', range(len(ACT_LAYERS)))
def test_against_reference_golden(index):
    name, kwargs, act_func = ACT_LAYERS[index]
    g = load_act_layer_golden()
    y, dx = run(getattr(attorch_b200, name)(**kwargs), g['x'], g['dy'])
    assert y.shape == g['x'].shape and y.dtype is torch.float32
    torch.testing.assert_close(y, g[f'y_{index:02d}_{name}_plain'], rtol=1e-4, atol=1e-5, equal_nan=True)
    torch.testing.assert_close(dx, g[f'dx_{index:02d}_{name}_plain'], rtol=1e-4, atol=1e-5, equal_nan=True)
    if oracle.parse_act_func(act_func)[0] not in oracle.FP32_ACTS | {'softsign'}:
        # Piecewise activations: bit-exact at the switch points (first 12 inputs of row 0).
        assert torch.equal(y[0, :12], g[f'y_{index:02d}_{name}_plain'][0, :12])
        assert torch.equal(dx[0, :12], g[f'dx_{index:02d}_{name}_plain'][0, :12])


@pytest.mark.parametrize('index', range(len(ACT_LAYERS)))
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_sixteen_bit_against_oracle(index, dtype):
    name, kwargs, act_func = ACT_LAYERS[index]
    gen = torch.Generator().manual_seed(index)
    x = (torch.randn(7, 333, generator=gen) * 2).to(dtype)       # 2331 elements: ragged tail
    dy = torch.randn(7, 333, generator=gen).to(dtype)
    y, dx = run(getattr(attorch_b200, name)(**kwargs), x, dy)
    assert y.dtype is dtype and dx.dtype is dtype
    torch.testing.assert_close(y.float(), oracle.act_layer_forward(x.float(), act_func).to(dtype).float(),
                               rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dx.float(), oracle.act_layer_backward(dy.float(), x.float(), act_func).to(dtype).float(),
                               rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize('label,drop_p', [('drop', 0.5), ('drop30', 0.3)])
@pytest.mark.parametrize('index', range(len(ACT_LAYERS)))
def test_dropout_against_reference_golden(index, label, drop_p):
    """
    Seeding Python's generator as the golden script did makes the layer draw the seed the reference
    drew; the same elements must then be dropped (integer work: bit-exact mask) and the kept ones
    must match the reference's values.
    """
    name, kwargs, act_func = ACT_LAYERS[index]
    g = load_act_layer_golden()
    tag = f'{index:02d}_{name}_{label}'
    random.seed(1000 + 3 * index + len(label))
    assert random.randint(0, 65535) == int(g[f'seed_{tag}'])
    random.seed(1000 + 3 * index + len(label))
    layer = getattr(attorch_b200, name)(drop_p=drop_p, **kwargs)
    layer.train()
    y, dx = run(layer, g['x'], g['dy'])
    ref_y, ref_dx = g[f'y_{tag}'], g[f'dx_{tag}']
    dropped = (oracle.dropout_uniform(int(g[f'seed_{tag}']), ref_y.numel()) < drop_p).view(ref_y.shape)
    assert torch.count_nonzero(y[dropped]) == 0 and torch.count_nonzero(dx[dropped]) == 0
    assert torch.equal((y != 0) | dropped, (ref_y != 0) | dropped)
    torch.testing.assert_close(y, ref_y, rtol=1e-4, atol=1e-5, equal_nan=True)
    torch.testing.assert_close(dx, ref_dx, rtol=1e-4, atol=1e-5, equal_nan=True)


@pytest.mark.parametrize('stream', ['reference', 'packed'])
@pytest.mark.parametrize('name,act_func', [('GELU', 'gelu'), ('ReLU', 'relu'), ('Tanh', 'tanh')])
@pytest.mark.parametrize('drop_p', [0.5, 0.1])
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_dropout_mask_is_the_oracles(name, act_func, drop_p, stream, dtype):
    """Integer work: the mask is bit-exact with the oracle's stream for the seed drawn, ragged tail included."""
    gen = torch.Generator().manual_seed(3)
    x = (torch.randn(5, 1001, generator=gen) + 0.1).to(dtype)
    dy = torch.randn(5, 1001, generator=gen).to(dtype)
    random.seed(11)
    seed = random.randint(0, 65535)          # what ActFuncAutoGrad will draw next
    random.seed(11)
    layer = getattr(attorch_b200, name)(drop_p=drop_p)
    layer.train()
    attorch_b200.set_dropout_stream(stream)
    try:
        y, dx = run(layer, x, dy)
    finally:
        attorch_b200.set_dropout_stream('reference')
    e_y = oracle.act_layer_forward(x.float(), act_func, drop_p, seed, stream)
    e_dx = oracle.act_layer_backward(dy.float(), x.float(), act_func, drop_p, seed, stream)
    dropped = (oracle.dropout_uniform(seed, x.numel(), stream) < drop_p).view(x.shape)
    assert torch.count_nonzero(y[dropped]) == 0 and torch.count_nonzero(dx[dropped]) == 0
    tol = dict(rtol=1e-4, atol=1e-5) if dtype is torch.float32 else dict(rtol=1e-2, atol=1e-2)
    assert torch.equal((y != 0) | dropped, (e_y.to(dtype) != 0) | dropped)
    torch.testing.assert_close(y.float(), e_y.to(dtype).float(), **tol)
    torch.testing.assert_close(dx.float(), e_dx.to(dtype).float(), **tol)
    assert abs(float(dropped.float().mean()) - drop_p) < 0.03


def test_dropout_streams_differ_and_repeat():
    x = torch.ones(4096, device=DEV)
    layer = attorch_b200.ReLU(drop_p=0.5)
    layer.train()
    masks = {}
    for stream in ('reference', 'packed', 'reference'):
        attorch_b200.set_dropout_stream(stream)
        random.seed(5)
        mask = layer(x) != 0
        attorch_b200.set_dropout_stream('reference')
        if stream in masks:
            assert torch.equal(masks[stream], mask)
        masks[stream] = mask
    assert not torch.equal(masks['reference'], masks['packed'])
    with pytest.raises(ValueError):
        attorch_b200.set_dropout_stream('triton')


def test_eval_mode_and_edge_shapes():
    layer = attorch_b200.GELU(drop_p=0.5)
    layer.eval()
    x = torch.randn(3, 5, 7)
    y = layer(x.to(DEV)).cpu()
    torch.testing.assert_close(y, torch.nn.functional.gelu(x), rtol=1e-4, atol=1e-5)
    assert attorch_b200.ReLU()(torch.empty(0, 4, device=DEV)).shape == (0, 4)
    # Non-contiguous input and an unaligned slice.
    base = torch.randn(10, 66, device=DEV)
    for view in (base[:, ::2], base.flatten()[3:300]):
        torch.testing.assert_close(attorch_b200.SiLU()(view), torch.nn.functional.silu(view), rtol=1e-4, atol=1e-5)
    with pytest.raises(RuntimeError):
        attorch_b200.GELU(approximate='fast')
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        attorch_b200.ReLU()(torch.randn(4))


@pytest.mark.parametrize('stream', ['reference', 'packed'])
def test_drop_everything(stream):
    """drop_p = 1: every element is dropped in both directions, as the reference's tl.where(random < 1, 0, ...) gives."""
    attorch_b200.set_dropout_stream(stream)
    try:
        layer = attorch_b200.GELU(drop_p=1.0)
        layer.train()
        y, dx = run(layer, torch.randn(5, 77).bfloat16(), torch.randn(5, 77))
    finally:
        attorch_b200.set_dropout_stream('reference')
    assert torch.count_nonzero(y) == 0 and torch.count_nonzero(dx) == 0
    assert not torch.isnan(y.float()).any() and not torch.isnan(dx.float()).any()
