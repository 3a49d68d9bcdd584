"""
Activation-function names of the fused linear layer and their ids in the CUDA library.

The names and the ``NAME_PARAM`` mini-language are those of the reference
(attorch/linear_layer.py:42-49 lists them, attorch/linear_layer.py:65-69 parses them); the ids
match ``enum Act`` in csrc/act_math.cuh and the AB200_ACT_* macros of include/attorch_b200.h.
"""

from typing import Optional, Tuple

ACT_IDS = {
    None: 0,
    'sigmoid': 1,
    'logsigmoid': 2,
    'tanh': 3,
    'relu': 4,
    'gelu': 5,
    'geluapprox': 6,
    'silu': 7,
    'relu6': 8,
    'hardsigmoid': 9,
    'hardtanh': 10,
    'hardswish': 11,
    'selu': 12,
    'mish': 13,
    'softplus': 14,
    'softsign': 15,
    'tanhshrink': 16,
    'leaky_relu': 17,
    'elu': 18,
    'celu': 19,
    'hardshrink': 20,
    'softshrink': 21,
}

# Activations that take the trailing ``_PARAM`` (negative slope, alpha, lambda).
PARAMETERIZED = frozenset({'leaky_relu', 'elu', 'celu', 'hardshrink', 'softshrink'})


def parse_act_func(act_func: Optional[str]) -> Tuple[Optional[str], Optional[float]]:
    """
    Splits an ``act_func`` string into its name and optional parameter.

    Same rule as the reference (attorch/linear_layer.py:65-69): if the string contains an
    underscore, the text after the last underscore is the parameter and must parse as a float,
    so ``'leaky_relu'`` on its own raises ``ValueError`` exactly as it does there. Unlike the
    reference, which only fails once the kernel is compiled, unknown names and a missing or
    superfluous parameter are rejected here with ``ValueError``.
    """
    if act_func is None:
        return None, None
    if not isinstance(act_func, str):
        raise TypeError(f'act_func must be a string or None, received {type(act_func).__name__}')

    name, param = act_func, None
    if '_' in act_func:
        comps = act_func.split('_')
        name = '_'.join(comps[:-1])
        param = float(comps[-1])

    if name not in ACT_IDS:
        raise ValueError(f'Unknown activation function {act_func!r}')
    if name in PARAMETERIZED and param is None:
        raise ValueError(f'Activation function {name!r} needs a parameter, e.g. {name}_0.01')
    if name not in PARAMETERIZED and param is not None:
        raise ValueError(f'Activation function {name!r} takes no parameter, received {act_func!r}')
    return name, param


def act_id(name: Optional[str]) -> int:
    """Id of a parsed activation name (``None`` is the identity)."""
    return ACT_IDS[name]
