"""
Pins the oracle's restatement of the standalone activation layers with fused dropout against
vectors produced by the reference's own layers (tests/golden/act_layers_fp32.npz) - dropout mask
included, for the seeds the reference drew - and the oracle's Philox restatement against the
library's host function.  No GPU needed.
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


@pytest.mark.parametrize('label,drop_p', [('drop', 0.5), ('drop30', 0.3)])
@pytest.mark.parametrize('index', range(len(ACT_LAYERS)))
def test_dropout_matches_reference_for_the_same_seed(index, label, drop_p):
    """
    The reference drew its mask with tl.rand from the seed stored beside each vector; the oracle's
    restatement of that generator must drop exactly the same elements, and kept elements are
    act(x) / (1 - p) (gradient: dy / (1 - p) * act'(x)).
    """
    name, _, act_func = ACT_LAYERS[index]
    g = load_act_layer_golden()
    tag = f'{index:02d}_{name}_{label}'
    seed = int(g[f'seed_{tag}'])
    ref_y, ref_dx = g[f'y_{tag}'], g[f'dx_{tag}']
    y = oracle.act_layer_forward(g['x'], act_func, drop_p, seed)
    dx = oracle.act_layer_backward(g['dy'], g['x'], act_func, drop_p, seed)
    dropped = (oracle.dropout_uniform(seed, g['x'].numel()) < drop_p).view(g['x'].shape)
    assert drop_p - 0.15 < dropped.float().mean() < drop_p + 0.15
    assert torch.count_nonzero(ref_y[dropped]) == 0 and torch.count_nonzero(ref_dx[dropped]) == 0
    plain_y = oracle.act_layer_forward(g['x'], act_func)
    assert torch.equal(ref_y != 0, ~dropped & (plain_y != 0))
    torch.testing.assert_close(y, ref_y, rtol=2e-5, atol=2e-5, equal_nan=True)
    torch.testing.assert_close(dx, ref_dx, rtol=2e-5, atol=2e-5, equal_nan=True)


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
        for stream, flags in (('reference', 0), ('packed', _lib.FLAG_DROPOUT_PACKED)):
            u = oracle.dropout_uniform(seed, 64, stream)
            for i in range(64):
                assert float(u[i]) == lib.ab200_dropout_uniform(seed, i, flags)
    # Known answer: Philox4x32-10 of counter 0 with key 0 (published test vector).
    import numpy as np
    words = oracle.philox4x32_10(np.array([0], dtype=np.uint64), 0)[0]
    assert [hex(int(w)) for w in words] == ['0x6627e8d5', '0xe169c58d', '0xbc57ac4c', '0x9b00dbd8']


@pytest.mark.parametrize('drop_p', [0.0, 1e-7, 0.1, 0.3, 0.5, 0.75, 0.999, 0.99999994])
def test_integer_threshold_equals_float_comparison(drop_p):
    """
    The kernels decide "dropped" by comparing the Philox word with an integer threshold; it must
    agree with the float comparison u < drop_p everywhere, checked on random words and on the
    words either side of the threshold.
    """
    import numpy as np
    from attorch_b200 import _lib
    from attorch_b200 import build as builder
    builder.build()
    lib = _lib.load()
    p32 = np.float32(drop_p)
    rng = np.random.default_rng(0)
    for flags in (0, _lib.FLAG_DROPOUT_PACKED):
        t = lib.ab200_dropout_threshold(float(p32), flags)
        near = np.clip(np.arange(-300, 300, dtype=np.int64) + t, 0, 2 ** 32 - 1).astype(np.uint64)
        words = np.concatenate([rng.integers(0, 2 ** 32, 20000, dtype=np.uint64), near,
                                np.array([0, 2 ** 31 - 1, 2 ** 31, 2 ** 32 - 1], dtype=np.uint64)])
        if flags:
            u = (words >> np.uint64(8)).astype(np.float32) / np.float32(16777216.0)
            m = words
        else:
            signed = words.astype(np.int64)
            signed = np.where(signed >= 2 ** 31, signed - 2 ** 32, signed)
            m = np.where(signed < 0, -signed - 1, signed).astype(np.uint64)
            u = m.astype(np.float32) * np.float32(4.6566127342e-10)
        assert np.array_equal(u < p32, m < np.uint64(t))


def test_drop_everything_in_the_oracle_and_on_the_host():
    """drop_p = 1 drops every element; probabilities outside [0, 1] are rejected with their own code."""
    import ctypes
    from attorch_b200 import _lib
    from attorch_b200 import build as builder
    x = torch.randn(64)
    assert torch.count_nonzero(oracle.act_layer_forward(x, 'relu', drop_p=1.0, seed=5)) == 0
    if not builder.LIB_PATH.exists():
        pytest.skip('library not built')
    lib = _lib.load()
    fake = ctypes.c_void_p(0x1000)
    assert lib.ab200_act_forward(fake, fake, 8, 2, 4, 0.0, 1.5, 0, None, 0) == -12
    assert lib.ab200_act_forward(fake, fake, 8, 2, 4, 0.0, -0.1, 0, None, 0) == -12
    assert lib.ab200_act_input_grad(fake, fake, fake, 0, 2, 4, 0.0, 1.0, 0, None, 0) == 0     # empty: nothing to do
