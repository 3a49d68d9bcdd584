"""
GPU parity of the element-wise kernels on bf16 data against the reference's own bf16 vectors
(tests/golden/elementwise_bf16.npz; see tests/test_elementwise_bf16_oracle.py for what those vectors
pin): the activation layers' forward and backward kernels, the linear layer's activation-backward
kernel (same arithmetic, plus the bias-gradient sums) and the gated linear unit.

The vectors hold the fp32 result with the low 16 bits dropped (the interpreter's conversion); the
kernels round to nearest even.  A correct kernel therefore returns either the vector's value or its
neighbour one bf16 step further from zero, except where the kernels' single-instruction exponential
and reciprocal (absolute error of a few 1e-7, which cancellation amplifies in x - tanh(x) near zero)
move a value across a rounding boundary: every element must be within one bf16 step plus 2e-6, and
at least 90 % must be one of the two expected values.
"""

import numpy as np
import pytest
import torch

import attorch_b200
from attorch_b200 import _lib
from attorch_b200.acts import act_id
from oracle import linear_oracle as oracle
from tests.helpers import ACT_LAYERS, GOLDEN_DIR

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def load():
    raw = np.load(GOLDEN_DIR / 'elementwise_bf16.npz')
    data = {k: torch.from_numpy(raw[k]) for k in raw.files if k != 'skipped'}
    return data, set(str(raw['skipped']).split(','))


def check(got, truncated, what):
    assert got.dtype is torch.bfloat16, what
    got = got.float().cpu()
    step = 2.0 ** -7 * truncated.abs() + 2e-6
    finite = ~torch.isnan(truncated)
    assert torch.equal(torch.isnan(got), ~finite), what
    assert bool(((got - truncated).abs()[finite] <= step[finite]).all()), f'{what}: more than one bf16 step off'
    away = got.abs() >= truncated.abs()             # the value itself or the next one away from zero
    assert float(away[finite].float().mean()) >= 0.9, what


@pytest.mark.parametrize('index', range(len(ACT_LAYERS)))
def test_activation_layer_kernels(index):
    name, kwargs, act_func = ACT_LAYERS[index]
    g, skipped = load()
    if f'{index:02d}_{name}' in skipped:
        pytest.skip('the reference could not produce this vector under the interpreter')
    x = g['x'].bfloat16().to(DEV).requires_grad_(True)
    y = getattr(attorch_b200, name)(**kwargs)(x)
    y.backward(g['dy'].bfloat16().to(DEV))
    check(y.detach(), g[f'y_{index:02d}_{name}'], f'{name} forward')
    check(x.grad, g[f'dx_{index:02d}_{name}'], f'{name} backward')


@pytest.mark.parametrize('index', range(len(ACT_LAYERS)))
def test_linear_layer_activation_backward_kernel(index):
    """ab200_act_backward (dZ = dY * act'(Z), with db) is the kernel the linear layer's backward runs."""
    name, _, act_func = ACT_LAYERS[index]
    g, skipped = load()
    if f'{index:02d}_{name}' in skipped:
        pytest.skip('the reference could not produce this vector under the interpreter')
    lib = _lib.load()
    act, param = oracle.parse_act_func(act_func)
    z = g['x'].bfloat16().to(DEV)
    dy = g['dy'].bfloat16().to(DEV)
    rows, cols = z.shape
    dz = torch.empty_like(z)
    db = torch.empty(cols, dtype=torch.float32, device=DEV)
    ws = torch.empty(max(lib.ab200_act_backward_workspace_bytes(rows, cols), 16), dtype=torch.uint8, device=DEV)
    _lib.check(lib.ab200_act_backward(dy.data_ptr(), z.data_ptr(), dz.data_ptr(), db.data_ptr(), rows, cols, cols, cols,
                                      cols, _lib.BF16, _lib.F32, act_id(act), param or 0.0, ws.data_ptr(), ws.numel(),
                                      torch.cuda.current_stream().cuda_stream), 'ab200_act_backward')
    torch.cuda.synchronize()
    check(dz, g[f'dx_{index:02d}_{name}'], f'{name} activation backward')
    torch.testing.assert_close(db.cpu(), dz.float().sum(0).cpu(), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize('act_func', [a for a in oracle.ALL_ACT_FUNCS if a is not None])
def test_gated_linear_unit_kernels(act_func):
    g, skipped = load()
    tag = act_func.replace('.', 'p')
    if f'glu_{tag}' in skipped or act_func.startswith('hardshrink'):
        pytest.skip('no usable reference vector (see tests/test_elementwise_bf16_oracle.py)')
    x = g['glu_x'].bfloat16().to(DEV).requires_grad_(True)
    y = attorch_b200.GLU(dim=-1, act_func=act_func)(x)
    y.backward(g['glu_dy'].bfloat16().to(DEV))
    check(y.detach(), g[f'glu_y_{tag}'], f'glu {act_func} forward')
    half = x.shape[-1] // 2
    check(x.grad[:, :half].contiguous(), g[f'glu_dx_{tag}'][:, :half].contiguous(), f'glu {act_func} backward, first half')
