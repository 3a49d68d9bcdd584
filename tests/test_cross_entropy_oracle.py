"""
Pins the oracle's restatement of the cross-entropy loss against vectors the reference's own layer
produced (tests/golden/cross_entropy_fp32.npz, made by tests/golden/make_golden.py under Triton's CPU
interpreter): loss and logits gradient, with and without class weights, for two upstream gradients.
No GPU needed.
"""

import numpy as np
import pytest
import torch

from oracle import linear_oracle as oracle
from tests.helpers import GOLDEN_DIR

CASES = 6


def load():
    raw = np.load(GOLDEN_DIR / 'cross_entropy_fp32.npz')
    return {k: torch.from_numpy(np.asarray(raw[k])) for k in raw.files}


@pytest.mark.parametrize('case', range(CASES))
def test_against_reference_vectors(case):
    g = load()
    x, target = g[f'x_{case}'], g[f'target_{case}']
    weight = g.get(f'weight_{case}')
    loss = oracle.cross_entropy_forward(x, target, weight)
    torch.testing.assert_close(loss, g[f'loss_{case}'], rtol=2e-6, atol=2e-6)
    for scale, label in ((1.0, 'unit'), (0.5, 'half')):
        dx = oracle.cross_entropy_backward(torch.tensor(scale), x, target, weight)
        torch.testing.assert_close(dx, g[f'dx_{case}_{label}'], rtol=2e-6, atol=2e-7)


def test_matches_pytorch_and_dtype_rule():
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(9, 31, generator=gen)
    t = torch.randint(0, 31, (9,), generator=gen)
    w = torch.rand(31, generator=gen) + 0.5
    torch.testing.assert_close(oracle.cross_entropy_forward(x, t), torch.nn.functional.cross_entropy(x, t))
    torch.testing.assert_close(oracle.cross_entropy_forward(x, t, w), torch.nn.functional.cross_entropy(x, t, w))
    assert oracle.cross_entropy_forward(x.bfloat16(), t).dtype is torch.bfloat16
    assert oracle.cross_entropy_forward(x.bfloat16(), t, autocast=True).dtype is torch.float32
    assert oracle.cross_entropy_backward(torch.tensor(1.0), x.half(), t, autocast=True).dtype is torch.float32


def test_module_surface_without_gpu():
    import attorch_b200
    loss = attorch_b200.CrossEntropyLoss()
    assert isinstance(loss, torch.nn.CrossEntropyLoss)
    with pytest.raises(RuntimeError, match='only supports averaging'):
        attorch_b200.CrossEntropyLoss(reduction='sum')
    with pytest.raises(RuntimeError, match='label smoothing'):
        attorch_b200.CrossEntropyLoss(label_smoothing=0.1)
    with pytest.raises(AssertionError, match='rank other than 2'):
        loss(torch.randn(4), torch.zeros(4, dtype=torch.long))
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        loss(torch.randn(4, 5), torch.zeros(4, dtype=torch.long))
    assert attorch_b200.nn.CrossEntropyLoss is attorch_b200.CrossEntropyLoss
