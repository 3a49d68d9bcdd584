"""
Pins the oracle's restatement of the standalone activation layers with fused dropout against
vectors produced by the reference's own layers (tests/golden/act_layers_fp32.npz), and the
oracle's Philox restatement against the library's host function.  No GPU needed.
"""

import pytest
import torch

from oracle import linear_oracle as oracle
from tests.helpers import ACT_LAYERS, load_act_layer_golden


@pytest.mark.parametrize('index', range(len(ACT_LAYERS)))
def test_act_layer_without_dropout(index):
    name, _, act_func = ACT_LAYERS[index]
    g = load_act_layer_golden()
    y = oracle.act_layer_forward(g['x'], act_func)
    dx = oracle.act_layer_backward(g['dy'], g['x'], act_func)
    torch.testing.assert_close(y, g[f'y_{index:02d}_{name}_plain'], rtol=2e-5, atol=2e-5, equal_nan=True)
    torch.testing.assert_close(dx, g[f'dx_{index:02d}_{name}_plain'], rtol=2e-5, atol=2e-5, equal_nan=True)


@pytest.mark.parametrize('index', range(len(ACT_LAYERS)))
def test_dropout_semantics_match_reference(index):
    """
    With drop_p = 0.5 the reference's mask comes from Triton's generator, so only the meaning of
    "dropped" and "kept" is compared: kept elements are act(x) / (1 - p), dropped ones are 0, and
    the gradient uses the same mask.  (As in the reference's own test, the mask is read off the
    reference's output; elements whose activation is 0 anyway are excluded.)
    """
    name, _, act_func = ACT_LAYERS[index]
    g = load_act_layer_golden()
    ref_y, ref_dx = g[f'y_{index:02d}_{name}_drop'], g[f'dx_{index:02d}_{name}_drop']
    plain_y = oracle.act_layer_forward(g['x'], act_func)
    plain_dx = oracle.act_layer_backward(g['dy'], g['x'], act_func)
    kept = ref_y != 0
    ambiguous = plain_y == 0
    assert 0.3 < kept[~ambiguous].float().mean() < 0.7
    torch.testing.assert_close(ref_y[kept], plain_y[kept] / 0.5, rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(ref_dx[kept], plain_dx[kept] / 0.5, rtol=2e-5, atol=2e-5)
    dropped = ~kept & ~ambiguous
    assert torch.count_nonzero(ref_dx[dropped]) == 0


def test_oracle_dropout_applies_its_own_mask():
    x = torch.randn(1000)
    u = oracle.dropout_uniform(123, 1000)
    y = oracle.act_layer_forward(x, 'relu', drop_p=0.3, seed=123)
    expect = torch.where(u < 0.3, torch.zeros(()), torch.relu(x) / 0.7)
    assert torch.equal(y, expect)
    assert 0.25 < (u < 0.3).float().mean() < 0.35


def test_philox_restatement_matches_library():
    from attorch_b200 import _lib
    from attorch_b200 import build as builder
    builder.build()
    lib = _lib.load()
    for seed in (0, 7, 65535):
        u = oracle.dropout_uniform(seed, 64)
        for i in range(64):
            assert float(u[i]) == lib.ab200_dropout_uniform(seed, i)
    # Known answer: Philox4x32-10 of counter 0 with key 0 (published test vector).
    import numpy as np
    words = oracle.philox4x32_10(np.array([0], dtype=np.uint64), 0)[0]
    assert [hex(int(w)) for w in words] == ['0x6627e8d5', '0xe169c58d', '0xbc57ac4c', '0x9b00dbd8']
