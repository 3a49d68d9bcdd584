"""
Interface with PyTorch fallback: every ``torch.nn`` name, with the modules this package implements
(``Linear``, ``LayerNorm``, ``GLU``, ``CrossEntropyLoss`` and the activation layers) taking the place of PyTorch's.  Same idea as the reference's
``attorch.nn`` (attorch/nn.py:6-8), so that ``from attorch_b200 import nn`` can replace
``from torch import nn`` in a model definition.  Mind the weight layout of ``Linear``
([in_features, out_features]); ``attorch_b200.convert`` moves parameters between the two layouts.
"""

from torch.nn import *  # noqa: F401,F403

from .act_layers import (CELU, ELU, GELU, SELU, Hardshrink, Hardsigmoid, Hardswish, Hardtanh,  # noqa: F401
                         LeakyReLU, LogSigmoid, Mish, ReLU, ReLU6, Sigmoid, SiLU, Softplus, Softshrink,
                         Softsign, Tanh, Tanhshrink)
from .cross_entropy_loss_layer import CrossEntropyLoss  # noqa: F401
from .glu_layer import GLU  # noqa: F401
from .layer_norm_layer import LayerNorm  # noqa: F401
from .linear_layer import Linear  # noqa: F401
