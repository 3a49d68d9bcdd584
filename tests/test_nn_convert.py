"""
The attorch.nn-style namespace (attorch/nn.py:6-8 of the reference) and the converters between
torch.nn.Linear's [out, in] weights and this package's [in, out].  Host logic only: no GPU needed.
"""

import torch

import attorch_b200
from attorch_b200 import convert, nn


def test_namespace_prefers_this_package_and_falls_back_to_torch():
    assert nn.Linear is attorch_b200.Linear
    assert nn.GELU is attorch_b200.GELU and nn.Softshrink is attorch_b200.Softshrink
    assert nn.LayerNorm is attorch_b200.LayerNorm and nn.CrossEntropyLoss is attorch_b200.CrossEntropyLoss
    assert nn.Conv2d is torch.nn.Conv2d and nn.BatchNorm2d is torch.nn.BatchNorm2d
    assert nn.Module is torch.nn.Module and nn.Parameter is torch.nn.Parameter


def test_module_round_trip():
    torch.manual_seed(0)
    ref = torch.nn.Linear(6, 6, bias=True)          # square: shapes cannot tell the layouts apart
    layer = convert.linear_from_torch(ref, act_func='relu')
    assert isinstance(layer, attorch_b200.Linear) and layer.act_func == 'relu'
    assert torch.equal(layer.weight, ref.weight.T) and layer.weight.is_contiguous()
    assert torch.equal(layer.bias, ref.bias)
    back = convert.linear_to_torch(layer)
    assert torch.equal(back.weight, ref.weight) and torch.equal(back.bias, ref.bias)
    no_bias = convert.linear_from_torch(torch.nn.Linear(3, 5, bias=False))
    assert no_bias.bias is None and no_bias.weight.shape == (3, 5)


def build(linear_cls, **kwargs):
    return torch.nn.Sequential(linear_cls(4, 8, **kwargs), torch.nn.ReLU(), linear_cls(8, 8, **kwargs))


def test_state_dict_conversion_both_ways():
    torch.manual_seed(1)
    torch_model = build(torch.nn.Linear)
    ours = build(attorch_b200.Linear, device='cpu')
    assert list(convert.linear_weight_keys(ours)) == ['0.weight', '2.weight']
    ours.load_state_dict(convert.convert_state_dict(torch_model.state_dict(), ours))
    assert torch.equal(ours[0].weight, torch_model[0].weight.T)
    assert torch.equal(ours[2].weight, torch_model[2].weight.T)
    assert torch.equal(ours[2].bias, torch_model[2].bias)
    restored = build(torch.nn.Linear)
    restored.load_state_dict(convert.convert_state_dict(ours.state_dict(), ours))
    for a, b in zip(restored.parameters(), torch_model.parameters()):
        assert torch.equal(a, b)


def test_swap_linear_layers_in_place():
    torch.manual_seed(2)
    model = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.Identity(),
                                torch.nn.Sequential(torch.nn.Linear(8, 2, bias=False)))
    weights = [model[0].weight.detach().clone(), model[2][0].weight.detach().clone()]
    convert.swap_linear_layers(model, act_funcs={'0': 'gelu'})
    assert isinstance(model[0], attorch_b200.Linear) and model[0].act_func == 'gelu'
    assert isinstance(model[2][0], attorch_b200.Linear) and model[2][0].act_func is None
    assert torch.equal(model[0].weight, weights[0].T) and torch.equal(model[2][0].weight, weights[1].T)


import pytest  # noqa: E402


@pytest.mark.gpu
def test_swapped_model_matches_pytorch_on_gpu():
    """A PyTorch MLP and its swapped copy (activation fused) agree, forward and backward."""
    torch.manual_seed(3)
    reference = torch.nn.Sequential(torch.nn.Linear(96, 160), torch.nn.GELU(), torch.nn.Linear(160, 64)).cuda()
    import copy
    swapped = copy.deepcopy(reference)
    convert.swap_linear_layers(swapped, act_funcs={'0': 'gelu'})
    swapped[1] = torch.nn.Identity()
    x = torch.randn(200, 96, device='cuda')
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    dy = torch.randn(200, 64, device='cuda')
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ya = reference(xa)
        ya.backward(dy)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = previous
    yb = swapped(xb)
    yb.backward(dy)
    attorch_b200.check_status()
    torch.testing.assert_close(yb, ya, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(xb.grad, xa.grad, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(swapped[0].weight.grad, reference[0].weight.grad.T, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(swapped[2].bias.grad, reference[2].bias.grad, rtol=1e-2, atol=1e-2)
