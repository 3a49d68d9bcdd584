"""
GPU parity of the gated linear unit (attorch_b200.GLU, through the C ABI) against the reference's
golden vectors and the CPU oracle.
"""

import pytest
import torch

import attorch_b200
from oracle import linear_oracle as oracle
from tests.helpers import glu_golden_cases, load_glu_golden

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def run(x, dy, dim, act_func):
    xg = x.to(DEV).requires_grad_(True)
    y = attorch_b200.GLU(dim=dim, act_func=act_func)(xg)
    y.backward(dy.to(DEV))
    return y.detach().cpu(), xg.grad.cpu()


@pytest.mark.parametrize('case,dim,act_func,tag', glu_golden_cases())
def test_against_reference_golden(case, dim, act_func, tag):
    g = load_glu_golden()
    y, dx = run(g[f'x_{case}'], g[f'dy_{case}'], dim, act_func)
    assert y.shape == g[f'y_{tag}'].shape and y.dtype is torch.float32
    torch.testing.assert_close(y, g[f'y_{tag}'], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dx, g[f'dx_{tag}'], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('shape,dim', [((64, 4096), -1), ((3, 50, 7), 1), ((130, 2), 1), ((2, 1000), 0),
                                       ((5, 16, 24), -1)])
@pytest.mark.parametrize('act_func', ['sigmoid', 'silu', 'gelu', 'leaky_relu_0.01'])
def test_against_oracle(shape, dim, act_func, dtype):
    """Vectorised (inner a multiple of 8) and ragged rows, every dtype."""
    gen = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(shape, generator=gen).to(dtype)
    out_shape = list(shape)
    out_shape[dim] //= 2
    dy = torch.randn(out_shape, generator=gen).to(dtype)
    y, dx = run(x, dy, dim, act_func)
    assert y.dtype is dtype and dx.dtype is dtype and dx.shape == x.shape
    tol = dict(rtol=1e-4, atol=1e-5) if dtype is torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(y.float(), oracle.glu_forward(x.float(), dim, act_func).to(dtype).float(), **tol)
    torch.testing.assert_close(dx.float(), oracle.glu_backward(dy.float(), x.float(), dim, act_func).to(dtype).float(),
                               **tol)


def test_edge_cases():
    layer = attorch_b200.GLU()
    assert layer.dim == -1 and layer.act_func == 'sigmoid'
    x = torch.randn(7, 12, device=DEV)
    torch.testing.assert_close(layer(x), torch.nn.functional.glu(x, -1), rtol=1e-4, atol=1e-5)
    # Non-contiguous input, empty input, odd extent, CPU tensor.
    base = torch.randn(12, 7, device=DEV)
    torch.testing.assert_close(layer(base.T), torch.nn.functional.glu(base.T, -1), rtol=1e-4, atol=1e-5)
    assert layer(torch.empty(0, 4, device=DEV)).shape == (0, 2)
    with pytest.raises(RuntimeError, match='must be even'):
        layer(torch.randn(3, 5, device=DEV))
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        layer(torch.randn(4, 4))
    # No gradient requested: nothing saved, forward still right.
    with torch.no_grad():
        assert layer(x).requires_grad is False
