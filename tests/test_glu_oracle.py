"""
Pins the oracle's restatement of the gated linear unit against vectors the reference's own layer
produced (tests/golden/glu_fp32.npz).  No GPU needed.
"""

import pytest
import torch

from oracle import linear_oracle as oracle
from tests.helpers import GLU_CASES, glu_golden_cases, load_glu_golden


@pytest.mark.parametrize('case,dim,act_func,tag', glu_golden_cases())
def test_glu_oracle_matches_reference(case, dim, act_func, tag):
    g = load_glu_golden()
    x, dy = g[f'x_{case}'], g[f'dy_{case}']
    assert tuple(x.shape) == GLU_CASES[case][0]
    torch.testing.assert_close(oracle.glu_forward(x, dim, act_func), g[f'y_{tag}'], rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(oracle.glu_backward(dy, x, dim, act_func), g[f'dx_{tag}'], rtol=2e-5, atol=2e-5)


def test_glu_oracle_agrees_with_pytorch():
    x = torch.randn(5, 12)
    torch.testing.assert_close(oracle.glu_forward(x, -1, 'sigmoid'), torch.nn.functional.glu(x, -1))
