"""
GPU tests of attorch_b200.GatedLinear (a projection with the gated linear unit fused into the GEMM's
epilogue, ab200_gated_linear_forward) against the composition it replaces,
attorch_b200.GLU(act_func)(attorch_b200.Linear(in, 2 * out)(x)) - bit for bit, forward and backward -
and against the CPU oracle of that composition (attorch/linear_layer.py:164-205 followed by
attorch/glu_layer.py:119-138 in the reference).
"""

import pytest
import torch

import attorch_b200
from attorch_b200 import _lib
from oracle import linear_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def build(k, h, bias, act_func, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    w = (torch.randn(k, 2 * h, generator=gen) / k ** 0.5).to(dtype)
    b = torch.randn(2 * h, generator=gen).to(dtype) if bias else None
    fused = attorch_b200.GatedLinear(k, h, bias=bias, act_func=act_func, device=DEV, dtype=dtype)
    plain = attorch_b200.Linear(k, 2 * h, bias=bias, device=DEV, dtype=dtype)
    with torch.no_grad():
        for layer in (fused, plain):
            layer.weight.copy_(w)
            if bias:
                layer.bias.copy_(b)
    return fused, plain, w, b


def run_both(m, k, h, bias, act_func, dtype, seed, flags=0, autocast=None):
    fused, plain, w, b = build(k, h, bias, act_func, dtype, seed)
    gen = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(m, k, generator=gen).to(dtype)
    dy = (torch.randn(m, h, generator=gen) * 0.02).to(autocast or dtype)
    results = []
    previous = attorch_b200.set_gemm_flags(flags)
    try:
        for which in ('fused', 'composed'):
            xg = x.to(DEV).requires_grad_(True)
            with torch.autocast('cuda', dtype=autocast or torch.bfloat16, enabled=autocast is not None):
                if which == 'fused':
                    y = fused(xg)
                    layer = fused
                else:
                    y = attorch_b200.GLU(dim=-1, act_func=act_func)(plain(xg))
                    layer = plain
            y.backward(dy.to(DEV))
            attorch_b200.check_status()
            results.append((y.detach().cpu(), xg.grad.cpu(), layer.weight.grad.cpu(),
                            layer.bias.grad.cpu() if bias else None))
    finally:
        attorch_b200.set_gemm_flags(previous)
    return results, x, w, b, dy


CASES = [(300, 264, 520, True), (1000, 512, 1024, False), (128, 64, 136, True), (2560, 320, 1408, True)]


@pytest.mark.parametrize('flags', [0, _lib.FLAG_NO_PAIR, _lib.FLAG_NO_TMA_STORE], ids=['pairs', 'single-cta', 'register-stores'])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('m,k,h,bias', CASES)
def test_equals_the_composition(m, k, h, bias, dtype, flags):
    (fused, composed), x, w, b, dy = run_both(m, k, h, bias, 'silu', dtype, seed=m + h, flags=flags)
    assert fused[0].shape == (m, h) and fused[0].dtype is dtype
    # Bit for bit where the composition's projection accumulates the same way (whole tiles).  Its small
    # fp32 cases and the ones with at most 128 rows take a stream-K schedule (atomic additions, another
    # order of summation); there the outputs agree to within that reordering.
    if dtype is not torch.float32 and m > 128:
        assert torch.equal(fused[0], composed[0]), 'output'
    else:
        torch.testing.assert_close(fused[0].float(), composed[0].float(), rtol=1e-5 if dtype is torch.float32 else 1e-2,
                                   atol=1e-5 if dtype is torch.float32 else 1e-2)
    # Backward runs the same kernels on the same stored halves in both; a small weight gradient may take
    # the stream-K schedule, whose atomic additions have no fixed order, so the gradients are compared to
    # within that reordering.
    # (fp32 operands are truncated to TF32 by the tensor cores: a last-bit difference in a stored half can
    # flip that truncation, 1e-3 relative per element of dZ.)
    tol = 2e-3 if dtype is torch.float32 else 1e-2
    for got, want, what in zip(fused[1:], composed[1:], ('dX', 'dW', 'db')):
        if want is None:
            assert got is None
        else:
            torch.testing.assert_close(got.float(), want.float(), rtol=tol, atol=tol, msg=lambda m: f'{what}: {m}')


@pytest.mark.parametrize('act_func', ['sigmoid', 'gelu', 'relu', 'silu', 'leaky_relu_0.01', 'tanh'])
def test_against_the_oracle(act_func):
    (fused, _), x, w, b, dy = run_both(384, 256, 392, True, act_func, torch.bfloat16, seed=9)
    z, _ = oracle.linear_forward(x, w, b, None)
    e_y = oracle.glu_forward(z, -1, act_func)
    torch.testing.assert_close(fused[0].float(), e_y.float(), rtol=1e-2, atol=1e-2)
    e_dz = oracle.glu_backward(dy, z, -1, act_func)
    e_dx, e_dw, _ = oracle.linear_backward(e_dz, x, None, w, None, torch.bfloat16, b)
    torch.testing.assert_close(fused[1].float(), e_dx.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(fused[2].float(), e_dw.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(fused[3].float(), e_dz.float().sum(0).bfloat16().float(), rtol=1e-2, atol=1e-2)


def test_autocast_and_three_dimensional_input():
    fused, plain, w, b = build(256, 320, True, 'silu', torch.float32, seed=3)
    x = torch.randn(4, 50, 256, device=DEV)
    with torch.autocast('cuda', dtype=torch.bfloat16):
        y = fused(x)
        ref = attorch_b200.GLU(dim=-1, act_func='silu')(plain(x))
    assert y.shape == (4, 50, 320) and y.dtype is torch.bfloat16
    assert torch.equal(y, ref)


def test_half_not_addressable_falls_back_to_two_kernels():
    """out_features = 100 (200 bytes per half in bf16: not a multiple of 16): the composition's two kernels run."""
    (fused, composed), *_ = run_both(96, 64, 100, True, 'gelu', torch.bfloat16, seed=5)
    assert torch.equal(fused[0], composed[0])
    for got, want in zip(fused[1:], composed[1:]):
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-3)
