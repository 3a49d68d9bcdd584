"""
Pins the oracle's restatement of layer normalisation against vectors the reference's own layer produced
(tests/golden/layer_norm.npz, made by tests/golden/make_golden.py under Triton's CPU interpreter): output,
input gradient, weight and bias gradients, fp32 and fp16, with and without the affine transform, 1-D to
3-D inputs, a shape the reference handles with several rows per program.  No GPU needed.
"""

import numpy as np
import pytest
import torch

from oracle import linear_oracle as oracle
from tests.helpers import GOLDEN_DIR, LAYER_NORM_BF16_CASES, LAYER_NORM_CASES, truncate_to_bf16


def load():
    raw = np.load(GOLDEN_DIR / 'layer_norm.npz')
    return {k: torch.from_numpy(np.asarray(raw[k])) for k in raw.files}


@pytest.mark.parametrize('case', range(len(LAYER_NORM_CASES)))
def test_against_reference_vectors(case):
    shape, dtype_name, affine, bias, eps = LAYER_NORM_CASES[case]
    dtype = getattr(torch, dtype_name)
    g = load()
    x, dy = g[f'x_{case}'], g[f'dy_{case}']
    assert tuple(x.shape) == shape and x.dtype is dtype
    w = g.get(f'w_{case}') if affine else None
    b = g.get(f'b_{case}') if affine and bias else None
    y, mean, inv_std = oracle.layer_norm_forward(x, w, b, eps)
    dx, dw, db = oracle.layer_norm_backward(dy, x, mean, inv_std, w, b is not None)
    assert y.dtype is dtype and dx.dtype is dtype
    # fp32: a few ulps of slack for the order of the row sums; fp16: one ulp of the stored value.
    tol = dict(rtol=1e-5, atol=1e-5) if dtype is torch.float32 else dict(rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(y, g[f'y_{case}'], **tol)
    torch.testing.assert_close(dx, g[f'dx_{case}'], **tol)
    if affine:
        # The reference adds its per-program partial sums in fp32 and the engine rounds to the parameter's dtype.
        scale = max(1.0, float(g[f'dw_{case}'].abs().max()))
        torch.testing.assert_close(dw.to(dtype), g[f'dw_{case}'], rtol=tol['rtol'], atol=tol['atol'] * scale)
        if bias:
            torch.testing.assert_close(db.to(dtype), g[f'db_{case}'], rtol=tol['rtol'], atol=tol['atol'] * scale)


def test_matches_pytorch():
    gen = torch.Generator().manual_seed(0)
    x = (torch.randn(7, 5, 48, generator=gen) * 2 + 1).requires_grad_(True)
    w, b = torch.randn(48, generator=gen).requires_grad_(True), torch.randn(48, generator=gen).requires_grad_(True)
    dy = torch.randn(7, 5, 48, generator=gen)
    ref = torch.nn.functional.layer_norm(x, (48,), w, b, 1e-5)
    ref.backward(dy)
    y, mean, inv_std = oracle.layer_norm_forward(x.detach(), w.detach(), b.detach(), 1e-5)
    dx, dw, db = oracle.layer_norm_backward(dy, x.detach(), mean, inv_std, w.detach(), True)
    torch.testing.assert_close(y, ref.detach(), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(dx, x.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dw, w.grad, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(db, b.grad, rtol=1e-5, atol=1e-4)
    assert oracle.layer_norm_forward(x.detach().bfloat16(), None, None)[0].dtype is torch.bfloat16
    assert oracle.layer_norm_forward(x.detach().half(), w, b, output_dtype=torch.float32)[0].dtype is torch.float32


def test_module_surface_without_gpu():
    import attorch_b200
    with pytest.raises(RuntimeError, match='must be an integer'):
        attorch_b200.LayerNorm((4, 8), device='cpu')
    norm = attorch_b200.LayerNorm(8, 1e-6, True, False, autocast_to_fp32=False, device='cpu')
    assert isinstance(norm, torch.nn.LayerNorm)
    assert norm.eps == 1e-6 and norm.bias is None and norm.weight.shape == (8,) and norm.autocast_to_fp32 is False
    assert list(norm.state_dict()) == ['weight']
    plain = attorch_b200.LayerNorm(8, elementwise_affine=False, device='cpu')
    assert plain.weight is None and plain.bias is None
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        norm(torch.randn(4, 8))
    assert attorch_b200.nn.LayerNorm is attorch_b200.LayerNorm
    fused = attorch_b200.LayerNormLinear(norm, attorch_b200.Linear(8, 16, act_func='gelu', device='cpu'))
    assert sorted(fused.state_dict()) == ['linear.bias', 'linear.weight', 'norm.weight']


@pytest.mark.parametrize('case', range(len(LAYER_NORM_BF16_CASES)))
def test_against_reference_bf16_vectors(case):
    """
    bf16 runs of the reference (tests/golden/layer_norm_bf16.npz).  The interpreter stores by truncation,
    so what is pinned is the oracle's fp32 value in front of the store: truncated the same way it equals the
    reference's output bit for bit, except where the two orders of the row sums put the fp32 value on
    different sides of a bf16 boundary (a handful of elements, then one bf16 step apart).
    """
    shape, param_dtype_name, bias = LAYER_NORM_BF16_CASES[case]
    raw = np.load(GOLDEN_DIR / 'layer_norm_bf16.npz')
    g = {k: torch.from_numpy(np.asarray(raw[k])) for k in raw.files if k.endswith(f'_{case}')}
    x, dy = g[f'x_{case}'].bfloat16(), g[f'dy_{case}'].bfloat16()
    w = g[f'w_{case}'].to(getattr(torch, param_dtype_name))
    b = g[f'b_{case}'].to(w.dtype) if bias else None
    y32, mean, inv_std = oracle.layer_norm_forward(x, w, b, output_dtype=torch.float32)
    dx32, dw32, db32 = oracle.layer_norm_backward(dy, x, mean, inv_std, w, bias, grad_dtype=torch.float32)
    for name, ours, ref in (('y', y32, g[f'y_{case}']), ('dx', dx32, g[f'dx_{case}'])):
        got = truncate_to_bf16(ours)
        same = (got == ref)
        assert same.float().mean() >= 0.995, name
        step = torch.maximum(ref.abs(), torch.tensor(1e-30)) * 2.0 ** -7          # one bf16 step, generously
        assert bool(((got - ref).abs() <= step)[~same].all()), name
    # Parameter gradients: fp32 sums, cast by the engine to the parameter's dtype (rounding to nearest).
    scale = max(1.0, float(g[f'dw_{case}'].abs().max()))
    tol = dict(rtol=1e-5, atol=1e-5 * scale) if w.dtype is torch.float32 else dict(rtol=8e-3, atol=8e-3 * scale)
    torch.testing.assert_close(dw32.to(w.dtype).float(), g[f'dw_{case}'], **tol)
    if bias:
        torch.testing.assert_close(db32.to(w.dtype).float(), g[f'db_{case}'], **tol)
