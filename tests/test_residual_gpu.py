"""
GPU tests of the residual add fused into the forward epilogue, Y = act(X W + b) + R
(attorch_b200.Linear.forward(input, residual), ab200_linear_forward_residual), on every kernel
family, against the oracle's forward plus the residual; the gradients of X, W, b must equal those of
the call without residual bit for bit (R does not enter them) and the gradient of R is dY.
"""

import pytest
import torch

import attorch_b200
from attorch_b200 import _lib
from oracle import linear_oracle as oracle
from tests.test_linear_gpu import FAMILIES, make_layer, seeded

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def assert_sum_close(y, unfused, residual):
    """
    y against unfused + residual, where `unfused` was rounded to the output dtype before the add: its
    rounding error (up to half a unit in the last place of ITS magnitude) survives a cancelling add,
    so the tolerance scales with the operands, not with the result.
    """
    bound = 1e-2 * (1 + unfused.float().abs() + residual.float().abs())
    error = (y.float() - (unfused.float() + residual.float())).abs()
    assert bool((error <= bound).all()), f'largest excess {float((error - bound).max())}'


def run(x, w, b, act_func, dy, residual, flags):
    layer = make_layer(w, b, act_func, w.dtype)
    xg = x.to(DEV).requires_grad_(True)
    rg = None if residual is None else residual.to(DEV).requires_grad_(True)
    previous = attorch_b200.set_gemm_flags(flags)
    try:
        y = layer(xg, rg) if rg is not None else layer(xg)
        y.backward(dy.to(DEV))
        attorch_b200.check_status()
    finally:
        attorch_b200.set_gemm_flags(previous)
    return (y.detach().cpu(), xg.grad.cpu(), layer.weight.grad.cpu(), layer.bias.grad.cpu(),
            None if rg is None else rg.grad.cpu())


@pytest.mark.parametrize('family,flags', FAMILIES)
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('shape,out_dim', [((1536, 320), 768), ((300, 264), 520), ((4, 50, 128), 96)])
@pytest.mark.parametrize('act_func', [None, 'gelu'])
def test_residual_in_the_epilogue(family, flags, dtype, shape, out_dim, act_func):
    x, w, b, dy = seeded(shape, out_dim, dtype, seed=31)
    gen = torch.Generator().manual_seed(32)
    residual = torch.randn((*shape[:-1], out_dim), generator=gen).to(dtype)
    y, dx, dw, db, dr = run(x, w, b, act_func, dy, residual, flags)
    y0, dx0, dw0, db0, _ = run(x, w, b, act_func, dy, None, flags)
    assert y.shape == y0.shape and y.dtype is dtype
    # Fused: one rounding of act(Z) + R; the caller's separate add would round twice.
    assert_sum_close(y, y0, residual)
    exact_fp32 = dtype is torch.float32 and family == 'generic'
    tf32 = 'truncate' if (dtype is torch.float32 and not exact_fp32) else None
    e_y, _ = oracle.linear_forward(x, w, b, act_func, None, tf32=tf32)
    assert_sum_close(y, e_y, residual)
    if family != 'streamk':          # atomically summed partials are not bit-repeatable
        assert torch.equal(dx, dx0) and torch.equal(dw, dw0) and torch.equal(db, db0)
    assert torch.equal(dr, dy)


def test_residual_of_another_dtype_and_layout():
    """An fp32, transposed residual under bf16 autocast is converted by the library's cast kernel."""
    x, w, b, dy = seeded((256, 128), 192, torch.float32, seed=33)
    layer = make_layer(w, b, 'silu', torch.float32)
    residual_t = torch.randn(192, 256, generator=torch.Generator().manual_seed(34))
    r = residual_t.to(DEV).T.requires_grad_(True)           # [256, 192], strides (1, 256)
    with torch.autocast('cuda', dtype=torch.bfloat16):
        y = layer(x.to(DEV), r)
        y_plain = layer(x.to(DEV))
    assert y.dtype is torch.bfloat16
    assert_sum_close(y.cpu(), y_plain.cpu(), residual_t.T.bfloat16())
    y.backward(dy.to(DEV).bfloat16())
    assert r.grad.dtype is torch.float32 and r.grad.shape == (256, 192)
    torch.testing.assert_close(r.grad, dy.to(DEV).bfloat16().float())
    with pytest.raises(AssertionError, match='residual'):
        layer(x.to(DEV), torch.zeros(256, 100, device=DEV))


def test_shared_out_last_round_with_residual():
    """The finishing kernel of the shared-out last round adds the residual too (90 pair tiles)."""
    x, w, b, dy = seeded((2560, 1024), 2304, torch.bfloat16, seed=35)
    residual = torch.randn(2560, 2304, generator=torch.Generator().manual_seed(36)).bfloat16()
    y, *_ = run(x, w, b, 'gelu', dy, residual, 0)
    y0, *_ = run(x, w, b, 'gelu', dy, None, 0)
    assert_sum_close(y, y0, residual)
