"""
ab200_linear_backward_input_fused (the activation gradient formed in the operand path of the input-gradient
product, A operand from tensor memory) against the arithmetic it stands for: dZ = dY (.) act'(Z) rounded to
bf16 as the separate pass rounds it (attorch/linear_layer.py:136-146 stores it in Z's dtype), then dZ * W^T
with fp32 accumulation (line 153), and against the library's own two kernels.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

# (M, K, N): one tile and one k-block; several tiles; ragged rows and output columns; more tiles than SMs.
SHAPES = [(128, 256, 64), (256, 512, 256), (300, 520, 192), (77, 40, 128), (4096, 2048, 512)]


@pytest.mark.parametrize('derivative_dtype', [torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize('dx_dtype', [torch.float32, torch.bfloat16], ids=str)
@pytest.mark.parametrize('M,K,N', SHAPES)
def test_fused_input_gradient(M, K, N, dx_dtype, derivative_dtype):
    from attorch_b200 import _lib
    lib = _lib.load()
    ids = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
    gen = torch.Generator().manual_seed(M + K + N)
    dy = (torch.randn(M, N, generator=gen) * 0.5).bfloat16()
    d = (torch.rand(M, N, generator=gen) * 1.2 - 0.1).to(derivative_dtype)
    w = (torch.randn(K, N, generator=gen) / N ** 0.5).bfloat16()
    dz = (dy.float() * d.float()).bfloat16()
    expected = dz.double() @ w.double().T
    dyg, dg, wg = dy.cuda(), d.cuda(), w.cuda()
    dx = torch.full((M, K), float('nan'), dtype=dx_dtype, device='cuda')
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.ab200_linear_backward_input_fused(dyg.data_ptr(), dg.data_ptr(), wg.data_ptr(), dx.data_ptr(), M, K, N,
                                                     N, N, N, K, ids[derivative_dtype], ids[dx_dtype], status.data_ptr(),
                                                     stream), 'ab200_linear_backward_input_fused')
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # fp32 accumulation of N products of magnitude <= max|dz| max|w|; bf16 output adds its rounding.
    scale = float(dz.float().abs().max() * w.float().abs().max()) * N ** 0.5
    tol = 2e-6 * N ** 0.5 * scale + (8e-3 * float(expected.abs().max()) if dx_dtype is torch.bfloat16 else 0.0)
    assert float((dx.cpu().double() - expected).abs().max()) <= max(tol, 1e-6)

    # The library's two kernels on the same operands.
    dz_gpu = torch.empty(M, N, dtype=torch.bfloat16, device='cuda')
    ws = torch.empty(max(lib.ab200_act_backward_workspace_bytes(M, N), 16), dtype=torch.uint8, device='cuda')
    act = _lib.ACT_SAVED_DERIVATIVE_F16 if derivative_dtype is torch.float16 else _lib.ACT_SAVED_DERIVATIVE
    _lib.check(lib.ab200_act_backward(dyg.data_ptr(), dg.data_ptr(), dz_gpu.data_ptr(), None, M, N, N, N, N, _lib.BF16,
                                      _lib.F32, act, 0.0, ws.data_ptr(), ws.numel(), stream), 'ab200_act_backward')
    torch.cuda.synchronize()
    assert torch.equal(dz_gpu.cpu(), dz)              # the transform warps round as this kernel does


def test_argument_checks():
    from attorch_b200 import _lib
    lib = _lib.load()
    t = torch.zeros(128, 128, dtype=torch.bfloat16, device='cuda')
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    call = lib.ab200_linear_backward_input_fused
    args = [t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 128, 128, 128, 128, 128, 128, 128, _lib.F16, _lib.BF16,
            status.data_ptr(), stream]
    bad = list(args); bad[6] = 100
    assert call(*bad) == -2                           # reduction length not a multiple of 64
    bad = list(args); bad[11] = _lib.F32
    assert call(*bad) == -3                           # fp32 derivative
    bad = list(args); bad[13] = None
    assert call(*bad) == -1                           # no status word
    bad = list(args); bad[0] = t.data_ptr() + 2
    assert call(*bad) == -5                           # unaligned dy
