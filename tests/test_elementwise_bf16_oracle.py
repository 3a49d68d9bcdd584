"""
Pins the oracle's arithmetic on bf16 data for the element-wise kernels (the activation layers, whose
backward is the kernel the linear layer's backward launches, and the gated linear unit) against bf16
vectors the reference itself produced (tests/golden/elementwise_bf16.npz, made by
tests/golden/make_golden.py under Triton's CPU interpreter).

What the vectors can and cannot pin: the interpreter converts fp32 to bf16 by dropping the low 16
bits, where a GPU rounds to nearest even.  So the vectors fix the fp32 value in front of the final
store - bit for bit, after the same truncation - for every activation, the piecewise ones included,
but not the rounding of the store itself; the oracle and the kernels round to nearest even there, as
Triton's fp32 -> bf16 conversion does on NVIDIA hardware.  Three activations are absent: the
interpreter of triton 3.6 cannot build the bf16 constants their kernels use (the file's 'skipped'
entry lists them).  No GPU needed.
"""

import numpy as np
import pytest
import torch

from oracle import linear_oracle as oracle
from tests.helpers import ACT_LAYERS, GOLDEN_DIR


def load():
    raw = np.load(GOLDEN_DIR / 'elementwise_bf16.npz')
    data = {k: torch.from_numpy(raw[k]) for k in raw.files if k != 'skipped'}
    return data, set(str(raw['skipped']).split(','))


def truncate_to_bf16(t):
    """fp32 -> bf16 as the interpreter does it: the low 16 bits dropped."""
    return (t.float().contiguous().view(torch.int32) & ~0xFFFF).view(torch.float32)


def assert_same(actual, expected, what):
    same = (actual == expected) | (torch.isnan(actual) & torch.isnan(expected))
    assert bool(same.all()), f'{what}: {int((~same).sum())} of {same.numel()} elements differ'


@pytest.mark.parametrize('index', range(len(ACT_LAYERS)))
def test_activation_layer_bf16(index):
    name, _, act_func = ACT_LAYERS[index]
    g, skipped = load()
    if f'{index:02d}_{name}' in skipped:
        pytest.skip('the reference could not produce this vector under the interpreter')
    x, dy = g['x'], g['dy']
    assert torch.equal(x.bfloat16().float(), x) and torch.equal(dy.bfloat16().float(), dy)   # bf16 numbers
    act, param = oracle.parse_act_func(act_func)
    y = oracle.act_forward(act, x, param)
    dx = dy * oracle.act_grad(act, x, param)
    assert_same(truncate_to_bf16(y), g[f'y_{index:02d}_{name}'], f'{name} forward')
    assert_same(truncate_to_bf16(dx), g[f'dx_{index:02d}_{name}'], f'{name} backward')
    # For the activations the reference evaluates in fp32 the oracle's own bf16 result is that value
    # rounded to nearest: never more than one bf16 step from the truncated one.  (The piecewise ones
    # the reference evaluates in bf16 arithmetic on a GPU, rounding after every operation, which the
    # interpreter does not do: for them the vectors pin the formula, not the intermediate roundings.)
    if act in oracle.FP32_ACTS:
        rounded = oracle.act_layer_forward(x.bfloat16(), act_func).float()
        expected = g[f'y_{index:02d}_{name}']
        ok = torch.isnan(expected) | ((rounded - expected).abs() <= 2.0 ** -7 * expected.abs())
        assert bool(ok.all())


@pytest.mark.parametrize('act_func', [a for a in oracle.ALL_ACT_FUNCS if a is not None])
def test_glu_bf16(act_func):
    """
    Output and the gradient of the first half.  The gradient of the second half, dy * x1 * act'(x2),
    starts with a product of two bf16 tensors, which the interpreter gets wrong (its stored values have
    magnitudes of 1e30); the same holds for everything hardshrink touches, whose kernel never
    widens to fp32.  Those entries of the file are not used.
    """
    g, skipped = load()
    tag = act_func.replace('.', 'p')
    if f'glu_{tag}' in skipped:
        pytest.skip('the reference could not produce this vector under the interpreter')
    if act_func.startswith('hardshrink'):
        pytest.skip('bf16 x bf16 products come out of the interpreter as garbage')
    x, dy = g['glu_x'], g['glu_dy']
    act, param = oracle.parse_act_func(act_func)
    x1, x2 = x.chunk(2, dim=-1)
    y = x1 * oracle.act_forward(act, x2, param)
    dx1 = dy * oracle.act_forward(act, x2, param)
    assert_same(truncate_to_bf16(y), g[f'glu_y_{tag}'], f'glu {act_func} forward')
    assert_same(truncate_to_bf16(dx1), g[f'glu_dx_{tag}'].chunk(2, dim=-1)[0], f'glu {act_func} backward, first half')
    garbage = g[f'glu_dx_{tag}'].chunk(2, dim=-1)[1]
    assert float(garbage.abs().max()) > 1e6 or act in ('relu', 'relu6', 'hardtanh', 'hardsigmoid')
