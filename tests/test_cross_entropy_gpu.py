"""
GPU parity of the cross-entropy loss (attorch_b200.CrossEntropyLoss, through the C ABI) against the
reference's golden vectors (fp32) and the CPU oracle (16-bit logits, autocast, large vocabularies,
strided logits, ragged and unaligned rows).
"""

import numpy as np
import pytest
import torch

import attorch_b200
from oracle import linear_oracle as oracle
from tests.helpers import GOLDEN_DIR

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def load():
    raw = np.load(GOLDEN_DIR / 'cross_entropy_fp32.npz')
    return {k: torch.from_numpy(np.asarray(raw[k])) for k in raw.files}


def run(x, target, weight=None, scale=1.0, autocast=None):
    xg = x.to(DEV).requires_grad_(True)
    layer = attorch_b200.CrossEntropyLoss(weight=None if weight is None else weight.to(DEV))
    with torch.autocast('cuda', dtype=autocast or torch.bfloat16, enabled=autocast is not None):
        loss = layer(xg, target.to(DEV))
    (loss * scale).backward()
    attorch_b200.check_status()
    return loss.detach().cpu(), xg.grad.cpu()


@pytest.mark.parametrize('case', range(6))
def test_against_reference_golden(case):
    g = load()
    x, target, weight = g[f'x_{case}'], g[f'target_{case}'], g.get(f'weight_{case}')
    for scale, label in ((1.0, 'unit'), (0.5, 'half')):
        loss, dx = run(x, target, weight, scale)
        assert loss.shape == () and loss.dtype is torch.float32 and dx.shape == x.shape
        torch.testing.assert_close(loss, g[f'loss_{case}'], rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(dx, g[f'dx_{case}_{label}'], rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize('weighted', [False, True])
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('batch,classes', [(33, 1000), (7, 50257), (256, 4099), (1, 3)])
def test_against_oracle(batch, classes, dtype, weighted):
    gen = torch.Generator().manual_seed(batch + classes)
    x = (torch.randn(batch, classes, generator=gen) * 4).to(dtype)
    target = torch.randint(0, classes, (batch,), generator=gen)
    weight = (torch.rand(classes, generator=gen) + 0.1) if weighted else None
    loss, dx = run(x, target, weight)
    assert loss.dtype is dtype and dx.dtype is dtype
    e_loss = oracle.cross_entropy_forward(x, target, weight)
    e_dx = oracle.cross_entropy_backward(torch.tensor(1.0), x, target, weight)
    tol = 1e-5 if dtype is torch.float32 else 1e-2
    torch.testing.assert_close(loss.float(), e_loss.float(), rtol=tol, atol=tol)
    torch.testing.assert_close(dx.float(), e_dx.float(), rtol=tol if dtype is not torch.float32 else 1e-4, atol=tol * 1e-2)
    # Each row of the gradient sums to zero (softmax minus one-hot), up to rounding.
    assert float(dx.float().sum(dim=1).abs().max()) < (1e-5 if dtype is torch.float32 else 2e-2)


def test_autocast_gives_fp32_loss_and_gradient():
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(48, 777, generator=gen).bfloat16()
    target = torch.randint(0, 777, (48,), generator=gen)
    loss, dx = run(x, target, autocast=torch.bfloat16)
    # The loss is fp32; the kernel writes an fp32 gradient too, which autograd then casts to the dtype of
    # the tensor it belongs to (as it does with the reference's).
    assert loss.dtype is torch.float32 and dx.dtype is torch.bfloat16
    torch.testing.assert_close(loss, oracle.cross_entropy_forward(x, target, autocast=True), rtol=1e-5, atol=1e-5)
    expected = oracle.cross_entropy_backward(torch.tensor(1.0), x, target, autocast=True)
    torch.testing.assert_close(dx.float(), expected.bfloat16().float(), rtol=1e-2, atol=1e-6)


def test_strided_logits_and_int32_targets():
    gen = torch.Generator().manual_seed(4)
    wide = torch.randn(20, 2 * 130, generator=gen)
    x = wide[:, ::2]                                   # stride 2 along the classes
    xt = torch.randn(130, 20, generator=gen).T         # stride 1 along the batch
    target = torch.randint(0, 130, (20,), generator=gen)
    for logits in (x, xt):
        xg = logits.to(DEV)
        if logits is x:
            xg = wide.to(DEV)[:, ::2]
        else:
            xg = xt.T.contiguous().to(DEV).T
        assert not xg.is_contiguous()
        xg.requires_grad_(True)
        loss = attorch_b200.CrossEntropyLoss()(xg, target.int().to(DEV))
        loss.backward()
        torch.testing.assert_close(loss.cpu(), oracle.cross_entropy_forward(logits, target), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(xg.grad.cpu(), oracle.cross_entropy_backward(torch.tensor(1.0), logits, target),
                                   rtol=1e-4, atol=1e-7)


def test_extreme_logits_do_not_overflow():
    x = torch.tensor([[1e4, -1e4, 0.0, 5.0], [-3e4, -3e4, -3e4, -3e4], [88.0, 89.0, 90.0, 91.0]])
    target = torch.tensor([0, 2, 3])
    loss, dx = run(x, target)
    assert torch.isfinite(loss) and torch.isfinite(dx).all()
    torch.testing.assert_close(loss, oracle.cross_entropy_forward(x, target), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(dx, oracle.cross_entropy_backward(torch.tensor(1.0), x, target), rtol=1e-4, atol=1e-7)


def test_projection_followed_by_the_loss():
    """The language-model head of the reference's example: Linear(n_embd -> vocab, no bias) then the loss."""
    gen = torch.Generator().manual_seed(6)
    tokens, n_embd, vocab = 96, 256, 1000
    h = torch.randn(tokens, n_embd, generator=gen).bfloat16()
    w = (torch.randn(n_embd, vocab, generator=gen) * 0.05).bfloat16()
    target = torch.randint(0, vocab, (tokens,), generator=gen)
    head = attorch_b200.Linear(n_embd, vocab, bias=False, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        head.weight.copy_(w)
    hg = h.to(DEV).requires_grad_(True)
    loss = attorch_b200.CrossEntropyLoss()(head(hg), target.to(DEV))
    loss.backward()
    attorch_b200.check_status()
    logits, _ = oracle.linear_forward(h, w, None, None)
    e_loss = oracle.cross_entropy_forward(logits, target)
    e_dlogits = oracle.cross_entropy_backward(torch.tensor(1.0), logits, target)
    torch.testing.assert_close(loss.float().cpu(), e_loss.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(head.weight.grad.float().cpu(), (h.float().T @ e_dlogits.float()), rtol=2e-2, atol=1e-3)
    torch.testing.assert_close(hg.grad.float().cpu(), e_dlogits.float() @ w.float().T, rtol=2e-2, atol=1e-4)
