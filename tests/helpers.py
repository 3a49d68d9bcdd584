"""Shared helpers of the test-suite: golden-vector loading and tolerances."""

from pathlib import Path
from typing import Dict, Optional

import numpy as np
import torch

GOLDEN_DIR = Path(__file__).resolve().parent / 'golden'

TORCH_DTYPES = {'float32': torch.float32, 'float16': torch.float16, 'bfloat16': torch.bfloat16}

# rtol = atol per dtype.  fp32 results of the reference (TF32 tensor-core products on a GPU, exact
# fp32 in its CPU interpreter) are compared at the tolerance the task states for TF32.
TOLERANCE = {torch.float32: 1e-2, torch.float16: 1e-2, torch.bfloat16: 1e-2}


def golden_names(prefix: str = ''):
    """Names of the linear-layer golden cases (the activation-layer and GLU files have their own loaders)."""
    return sorted(p.stem for p in GOLDEN_DIR.glob(f'{prefix}*.npz')
                  if not p.stem.startswith(('act_layers', 'glu_', 'elementwise_', 'cross_entropy_', 'layer_norm')))


# (module name, constructor arguments, act_func string) in the order of tests/golden/make_golden.py.
ACT_LAYERS = [('Sigmoid', {}, 'sigmoid'), ('LogSigmoid', {}, 'logsigmoid'), ('Tanh', {}, 'tanh'),
              ('ReLU', {}, 'relu'), ('GELU', {}, 'gelu'), ('GELU', {'approximate': 'tanh'}, 'geluapprox'),
              ('SiLU', {}, 'silu'), ('ReLU6', {}, 'relu6'), ('Hardsigmoid', {}, 'hardsigmoid'),
              ('Hardtanh', {}, 'hardtanh'), ('Hardswish', {}, 'hardswish'), ('SELU', {}, 'selu'),
              ('Mish', {}, 'mish'), ('Softplus', {}, 'softplus'), ('Softsign', {}, 'softsign'),
              ('Tanhshrink', {}, 'tanhshrink'), ('LeakyReLU', {'negative_slope': 0.01}, 'leaky_relu_0.01'),
              ('ELU', {'alpha': 1.0}, 'elu_1.0'), ('CELU', {'alpha': 1.0}, 'celu_1.0'),
              ('Hardshrink', {'lambd': 0.5}, 'hardshrink_0.5'), ('Softshrink', {'lambd': 0.5}, 'softshrink_0.5')]


def load_act_layer_golden():
    """The reference's activation-layer vectors: dict of torch tensors keyed as in the .npz."""
    raw = np.load(GOLDEN_DIR / 'act_layers_fp32.npz')
    return {key: torch.from_numpy(raw[key]) for key in raw.files}


def config1_inputs():
    """The smallest configuration (fp32, 64 x 128 -> 256, bias, relu) inputs, regenerated as tests/golden/make_golden.py makes them."""
    torch.manual_seed(0)
    x = torch.randn(64, 128)
    torch.manual_seed(0)
    linear = torch.nn.Linear(128, 256, bias=True)
    w = linear.weight.detach().T.contiguous()
    b = linear.bias.detach().clone()
    torch.manual_seed(0)
    dy = torch.randn(64, 256)
    return x, w, b, dy


def load_golden(name: str) -> Dict[str, Optional[torch.Tensor]]:
    """Loads one golden case: tensors in their dtype, plus 'act_func' and 'dtype'."""
    raw = np.load(GOLDEN_DIR / f'{name}.npz')
    dtype = TORCH_DTYPES[str(raw['dtype'])]
    act_func = str(raw['act_func'])
    case = {'act_func': None if act_func == 'None' else act_func, 'dtype': dtype}
    if 'x' in raw:
        for key in ('x', 'w', 'b', 'dy'):
            arr = raw[key]
            case[key] = None if arr.size == 0 else torch.from_numpy(arr).to(dtype)
    else:
        assert name.startswith('config1')
        case['x'], case['w'], case['b'], case['dy'] = config1_inputs()
    for key in ('y', 'dx', 'dw', 'db'):
        arr = raw[key]
        case[key] = None if arr.size == 0 else torch.from_numpy(arr).to(dtype)
    case['input_checksum'] = str(raw['input_checksum'])
    return case


def assert_close(actual: torch.Tensor, expected: torch.Tensor, tol: float, what: str) -> None:
    assert actual.shape == expected.shape, f'{what}: shape {actual.shape} vs {expected.shape}'
    assert actual.dtype == expected.dtype, f'{what}: dtype {actual.dtype} vs {expected.dtype}'
    torch.testing.assert_close(actual.float().cpu(), expected.float().cpu(), rtol=tol, atol=tol,
                               equal_nan=True, msg=lambda m: f'{what}: {m}')


# (input shape, gated dimension) of the cases in tests/golden/glu_fp32.npz; case 0 holds every
# activation setting, the others sigmoid, gelu and relu (tests/golden/make_golden.py: GLU_CASES).
GLU_CASES = [((6, 10), -1), ((6, 10), 0), ((4, 6, 5), 1), ((2, 3, 8), 2), ((2, 4, 3, 2), -3)]


def glu_golden_cases():
    """[(case index, gated dimension, act_func, tag)] for every vector pair in glu_fp32.npz."""
    from oracle.linear_oracle import ALL_ACT_FUNCS
    cases = []
    for case, (_, dim) in enumerate(GLU_CASES):
        acts = [a for a in ALL_ACT_FUNCS if a is not None] if case == 0 else ['sigmoid', 'gelu', 'relu']
        cases += [(case, dim, act, f'{case}_{act.replace(".", "p")}') for act in acts]
    return cases


def load_glu_golden():
    raw = np.load(GOLDEN_DIR / 'glu_fp32.npz')
    return {key: torch.from_numpy(raw[key]) for key in raw.files}


# (shape, dtype, elementwise_affine, bias, eps) in the order of tests/golden/make_golden.py.
LAYER_NORM_CASES = [
    ((16,), 'float32', True, True, 1e-5),
    ((5, 40), 'float32', True, True, 1e-5),
    ((5, 40), 'float32', True, False, 1e-6),
    ((5, 40), 'float32', False, False, 1e-5),
    ((3, 7, 96), 'float32', True, True, 1e-5),
    ((2049, 2), 'float32', True, True, 1e-5),
    ((257, 33), 'float32', True, True, 1e-5),
    ((6, 1100), 'float32', True, True, 1e-5),
    ((4, 6, 64), 'float16', True, True, 1e-5),
    ((9, 200), 'float16', True, False, 1e-5),
    ((9, 200), 'float16', False, False, 1e-6),
]

# (shape, parameter dtype, bias): the bf16 layer-normalisation cases of tests/golden/make_golden.py.
LAYER_NORM_BF16_CASES = [
    ((7, 40), 'bfloat16', True),
    ((33, 200), 'bfloat16', False),
    ((4, 6, 64), 'float32', True),
    ((5, 1040), 'bfloat16', True),
]


def truncate_to_bf16(t):
    """fp32 -> bf16 by dropping the low 16 bits, as Triton's CPU interpreter stores (a GPU rounds to nearest)."""
    import torch
    return (t.float().contiguous().view(torch.int32) & -65536).view(torch.float32)
