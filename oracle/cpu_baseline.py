"""
TEST / BENCHMARK INFRASTRUCTURE - the CPU timing baseline of the fused linear layer.  Not part of
the product: only ``bench.py``'s CPU-baseline legs import it.

What is timed is the CPU computation the reference's own test compares attorch.Linear against:
``torch.nn.Linear`` followed by ``torch.nn.functional.<act>``, forward and backward
(tests/test_linear_layer.py:44-56 of the reference), on all host cores.  The reference's Triton
kernels themselves run on a CPU only inside Triton's Python interpreter, which is a correctness
tool (seconds for a 64 x 128 x 256 layer), not a timing baseline.
"""

import os
import time
from typing import Dict, Optional

import torch
import torch.nn.functional as F


def _activation(act_func: Optional[str]):
    if act_func is None:
        return lambda t: t
    name, _, param = act_func.rpartition('_') if '_' in act_func else (act_func, '', '')
    if name == 'geluapprox':
        return lambda t: F.gelu(t, approximate='tanh')
    fn = getattr(F, name)
    return (lambda t: fn(t, float(param))) if param else fn


def time_torch_cpu_linear(rows: int, in_features: int, out_features: int, act_func: Optional[str],
                          bias: bool, autocast_dtype: Optional[torch.dtype], steps: int,
                          warmup: int) -> Dict[str, float]:
    """
    Times ``steps`` forward+backward passes of nn.Linear + activation on ``rows`` input rows.
    Returns seconds per step, the thread count used and the TFLOP/s at 6 * rows * in * out
    floating-point operations per step (the three products; bias and activation not counted).
    """
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    layer = torch.nn.Linear(in_features, out_features, bias=bias)
    act = _activation(act_func)
    x = torch.randn(rows, in_features, requires_grad=True)
    dy = torch.randn(rows, out_features) * 0.01

    def step():
        x.grad = None
        layer.zero_grad(set_to_none=True)
        with torch.autocast('cpu', dtype=autocast_dtype or torch.bfloat16,
                            enabled=autocast_dtype is not None):
            y = act(layer(x))
        y.backward(dy.to(y.dtype))

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    seconds = (time.perf_counter() - t0) / max(steps, 1)
    flops = 6.0 * rows * in_features * out_features
    return {'seconds_per_step': seconds, 'threads': threads, 'tflops': flops / seconds / 1e12}
