"""
Pins the CPU oracle (oracle/linear_oracle.py) against golden vectors produced by the reference
itself (tests/golden/make_golden.py).  No GPU needed.
"""

import hashlib

import numpy as np
import pytest
import torch

from oracle import linear_oracle as oracle
from tests.helpers import assert_close, golden_names, load_golden


def _np(t):
    return np.zeros(0, dtype=np.float32) if t is None else t.numpy()


@pytest.mark.parametrize('name', golden_names())
def test_oracle_matches_reference_golden(name):
    case = load_golden(name)
    # The inputs the test uses are bit-identical to the ones the reference was run on.
    h = hashlib.sha256()
    for key in ('x', 'w', 'b', 'dy'):
        h.update(np.ascontiguousarray(_np(case[key])).tobytes())
    assert h.hexdigest() == case['input_checksum'], 'golden inputs changed'

    y, pre_act, dx, dw, db = oracle.linear_forward_backward(
        case['x'], case['w'], case['b'], case['act_func'], case['dy'])
    # fp32: the interpreter and the oracle both use exact fp32 products, so only summation order
    # and transcendental implementations differ.  fp16: one rounding step of slack.
    tol = 2e-5 if case['dtype'] is torch.float32 else 2e-3
    assert_close(y, case['y'], tol, 'output')
    # The reference's fp16 backward products ran as CPU fp16 matmuls here (its torch.autocast('cuda')
    # does nothing for CPU tensors), whose accumulation differs from the GPU's by an fp16 ulp or so.
    tol = 2e-5 if case['dtype'] is torch.float32 else 1e-2
    assert_close(dx, case['dx'], tol, 'input grad')
    assert_close(dw, case['dw'], tol, 'weight grad')
    if case['b'] is not None:
        assert_close(db, case['db'], tol, 'bias grad')
    else:
        assert db is None


@pytest.mark.parametrize('name', golden_names('switch_'))
def test_switch_points_exact(name):
    """At the piecewise switch points the oracle reproduces the reference bit for bit."""
    case = load_golden(name)
    if case['act_func'] is not None and case['act_func'].split('_')[0] in (
            'sigmoid', 'logsigmoid', 'tanh', 'gelu', 'geluapprox', 'silu', 'selu', 'mish', 'softplus',
            'tanhshrink', 'elu', 'celu'):
        pytest.skip('smooth activation: no switch point')
    y, _, dx, _, _ = oracle.linear_forward_backward(
        case['x'], case['w'], case['b'], case['act_func'], case['dy'])
    assert torch.equal(y, case['y'])
    assert torch.equal(dx, case['dx'])


def test_oracle_matches_torch_on_config1():
    """The smallest configuration (fp32, 64 x 128 -> 256, bias, relu) against torch.nn.Linear + ReLU, the comparator of the reference's test."""
    case = load_golden('config1_fp32_relu')
    x = case['x'].clone().requires_grad_(True)
    lin = torch.nn.Linear(128, 256)
    with torch.no_grad():
        lin.weight.copy_(case['w'].T)
        lin.bias.copy_(case['b'])
    y_ref = torch.relu(lin(x))
    y_ref.backward(case['dy'])
    y, _, dx, dw, db = oracle.linear_forward_backward(case['x'], case['w'], case['b'], 'relu', case['dy'])
    assert_close(y, y_ref.detach(), 1e-5, 'output')
    assert_close(dx, x.grad, 1e-5, 'dx')
    assert_close(dw, lin.weight.grad.T.contiguous(), 1e-4, 'dw')
    assert_close(db, lin.bias.grad, 1e-4, 'db')


@pytest.mark.parametrize('act_func', oracle.ALL_ACT_FUNCS)
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_oracle_matches_torch_functional(act_func, dtype):
    """The restated activation math against torch.nn.functional, the reference tests' comparator."""
    import torch.nn.functional as F
    torch.manual_seed(0)
    x = torch.randn(16, 24).to(dtype)
    w = (torch.randn(24, 40) / 5).to(dtype)
    b = torch.randn(40).to(dtype)
    y, _ = oracle.linear_forward(x, w, b, act_func)
    z = (x.float() @ w.float() + b.float())
    if act_func is None:
        expect = z
    else:
        name, param = oracle.parse_act_func(act_func)
        fn = {'geluapprox': lambda t: F.gelu(t, approximate='tanh')}.get(name, getattr(F, name, None))
        expect = fn(z) if param is None else fn(z, param)
    tol = 1e-5 if dtype is torch.float32 else 1e-2
    torch.testing.assert_close(y.float(), expect.to(dtype).float(), rtol=tol, atol=tol)


def test_dtype_rule():
    assert oracle.output_dtype_rule(torch.float32, None) is torch.float32
    assert oracle.output_dtype_rule(torch.float32, torch.float16) is torch.float16
    assert oracle.output_dtype_rule(torch.float16, torch.float16) is torch.float16
    assert oracle.output_dtype_rule(torch.float32, torch.bfloat16) is torch.bfloat16
    assert oracle.output_dtype_rule(torch.bfloat16, None) is torch.bfloat16


def test_tf32_round():
    x = torch.tensor([1.0, 1.0 + 2 ** -11, 1.0 + 2 ** -10, 3.14159265, 1 + 3 * 2 ** -12])
    r = oracle.tf32_round(x)
    assert r[0] == 1.0 and r[2] == 1.0 + 2 ** -10 and r[4] == 1.0 + 2 ** -10
    assert abs(float(r[3]) - 3.14159265) < 3.2 * 2 ** -11
    assert (r.view(torch.int32) & 0x1FFF).eq(0).all()
    t = oracle.tf32_round(x, 'truncate')
    assert t[0] == 1.0 and t[1] == 1.0 and t[2] == 1.0 + 2 ** -10 and t[4] == 1.0
    assert (t.abs() <= x.abs()).all()
