"""
Moving parameters between ``torch.nn.Linear`` (weight ``[out_features, in_features]``) and this
package's ``Linear`` (weight ``[in_features, out_features]``, the reference's layout,
attorch/linear_layer.py:170-173 and 200): module converters and a state_dict converter for
checkpoints written by PyTorch models.
"""

from typing import Dict, Iterable, Optional

import torch
from torch import Tensor, nn

from .linear_layer import Linear


def linear_from_torch(module: nn.Linear, act_func: Optional[str] = None) -> Linear:
    """
    A ``Linear`` with the parameters of ``module`` (values copied, weight transposed), on its device
    and in its dtype, optionally fusing ``act_func``.
    """
    if not isinstance(module, nn.Linear) or isinstance(module, Linear):
        raise TypeError(f'expected a torch.nn.Linear, received {type(module).__name__}')
    layer = Linear(module.in_features, module.out_features, bias=module.bias is not None, act_func=act_func,
                   device=module.weight.device, dtype=module.weight.dtype)
    with torch.no_grad():
        layer.weight.copy_(module.weight.T)
        if module.bias is not None:
            layer.bias.copy_(module.bias)
    layer.weight.requires_grad_(module.weight.requires_grad)
    if module.bias is not None:
        layer.bias.requires_grad_(module.bias.requires_grad)
    return layer


def linear_to_torch(layer: Linear) -> nn.Linear:
    """The ``torch.nn.Linear`` with the parameters of ``layer``; a fused activation is not carried over."""
    if not isinstance(layer, Linear):
        raise TypeError(f'expected an attorch_b200.Linear, received {type(layer).__name__}')
    module = nn.Linear(layer.in_features, layer.out_features, bias=layer.bias is not None,
                       device=layer.weight.device, dtype=layer.weight.dtype)
    with torch.no_grad():
        module.weight.copy_(layer.weight.T)
        if layer.bias is not None:
            module.bias.copy_(layer.bias)
    return module


def linear_weight_keys(model: nn.Module) -> Iterable[str]:
    """state_dict keys of the weights of every ``Linear`` of this package inside ``model``."""
    for name, module in model.named_modules():
        if isinstance(module, Linear):
            yield f'{name}.weight' if name else 'weight'


def convert_state_dict(state_dict: Dict[str, Tensor], model: nn.Module) -> Dict[str, Tensor]:
    """
    A copy of ``state_dict`` (written by the same architecture built from ``torch.nn.Linear``) in
    which the weight of every ``Linear`` of ``model`` is transposed, ready for
    ``model.load_state_dict``.  The keys decide, not the shapes, so square weights are handled too.
    Applying it to a state_dict of ``model`` itself gives the PyTorch layout back.
    """
    converted = dict(state_dict)
    for key in linear_weight_keys(model):
        if key in converted:
            converted[key] = converted[key].T.contiguous()
    return converted


def swap_linear_layers(model: nn.Module, act_funcs: Optional[Dict[str, str]] = None) -> nn.Module:
    """
    Replaces, in place, every ``torch.nn.Linear`` inside ``model`` with this package's ``Linear``
    holding the same parameters.  ``act_funcs`` maps module names (as in ``named_modules``) to an
    activation to fuse into that layer; the caller removes the standalone activation that follows it.
    """
    act_funcs = act_funcs or {}
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            if isinstance(child, nn.Linear) and not isinstance(child, Linear):
                full = f'{name}.{child_name}' if name else child_name
                setattr(module, child_name, linear_from_torch(child, act_funcs.get(full)))
    return model
