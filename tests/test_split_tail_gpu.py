"""
GPU tests of the schedule that runs the last round of output tiles as half-width units
(ab200_last_schedule() == 3; the default where it pays, see launch_cfg in csrc/gemm_launch.cuh), called
through the C ABI for each of the three GEMMs of the layer:
forward (A K-major, B MN-major), dX (both K-major), dW (both MN-major).  Results are compared with
float64 products of the same (rounded) operands and, bit for bit, with the whole-tile schedule:
both run the same tcgen05 instructions per output element in the same order.
"""

import os

import pytest
import torch

from attorch_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = 'cuda'


@pytest.fixture(autouse=True)
def default_tail_mode():
    os.environ.pop('AB200_TAIL_MODE', None)
    yield
    os.environ.pop('AB200_TAIL_MODE', None)

IDS = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def reference_product(a, b):
    return (a.double().cpu() @ b.double().cpu())


def tf32(t):
    return (t.view(torch.int32) & ~0x1FFF).view(torch.float32) if t.dtype is torch.float32 else t


def run(which, M, K, N, dtype, flags):
    """One GEMM of a layer with M tokens, K inputs, N outputs; returns (result, expected, schedule)."""
    lib = _lib.load()
    gen = torch.Generator(device=DEV).manual_seed(M + K + N)
    x = torch.randn(M, K, device=DEV, generator=gen).to(dtype)
    w = (torch.randn(K, N, device=DEV, generator=gen) / K ** 0.5).to(dtype)
    dz = torch.randn(M, N, device=DEV, generator=gen).to(dtype)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    dt = IDS[dtype]
    flags |= _lib.FLAG_FORCE_TCGEN05 | _lib.FLAG_NO_STREAMK
    if which == 'fwd':
        bias = torch.randn(N, device=DEV, generator=gen).to(dtype)
        out = torch.empty(M, N, device=DEV, dtype=dtype)
        pre = torch.empty(M, N, device=DEV, dtype=dtype)
        _lib.check(lib.ab200_linear_forward(x.data_ptr(), w.data_ptr(), bias.data_ptr(), pre.data_ptr(), out.data_ptr(),
                                            M, K, N, K, 1, N, 1, N, N, dt, dt, dt, 4, 0.0, None, 0,
                                            status.data_ptr(), stream, flags), 'forward')       # act 4 = relu
        expected = torch.relu(reference_product(tf32(x), tf32(w)) + bias.double().cpu())
        got = out
        # The saved pre-activation must be consistent with the output.
        assert torch.equal(torch.relu(pre.float()).to(dtype)[pre > 0], out[pre > 0])
    elif which == 'dx':
        out = torch.empty(M, K, device=DEV, dtype=dtype)
        _lib.check(lib.ab200_linear_backward_input(dz.data_ptr(), w.data_ptr(), out.data_ptr(), M, K, N, N, 1, N, 1, K,
                                                   dt, dt, None, 0, status.data_ptr(), stream, flags), 'dx')
        expected = reference_product(tf32(dz), tf32(w).T)
        got = out
    else:
        out = torch.empty(K, N, device=DEV, dtype=dtype)
        _lib.check(lib.ab200_linear_backward_weight(x.data_ptr(), dz.data_ptr(), out.data_ptr(), M, K, N, K, 1, N, 1, N,
                                                    dt, dt, None, 0, status.data_ptr(), stream, flags), 'dw')
        expected = reference_product(tf32(x).T, tf32(dz))
        got = out
    schedule = lib.ab200_last_schedule()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return got.cpu(), expected, schedule


def sms():
    return torch.cuda.get_device_properties(0).multi_processor_count


# (which, M, K, N): output tiles of 256 x 256 (CTA pairs) number 110 = 74 + 36 on 148 SMs.
PAIR_CASES = [('fwd', 2560, 512, 2816), ('dx', 2560, 2816, 512), ('dw', 512, 2560, 2816),
              ('fwd', 2560, 520, 2800)]       # ragged last column tile, K not a multiple of 64


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('which,M,K,N', PAIR_CASES)
def test_half_width_last_round_pairs(which, M, K, N, dtype):
    if sms() != 148:
        pytest.skip('tile counts are chosen for 148 SMs')
    got, expected, schedule = run(which, M, K, N, dtype, 0)
    assert schedule == 3
    whole, _, whole_schedule = run(which, M, K, N, dtype, _lib.FLAG_WHOLE_TILES)
    assert whole_schedule == 0
    assert torch.equal(got, whole)
    tol = 2e-2 if dtype is torch.bfloat16 else 2e-3
    torch.testing.assert_close(got.double(), expected, rtol=tol, atol=tol)


@pytest.mark.parametrize('which,M,K,N', [('fwd', 2560, 512, 2816), ('dx', 2560, 2816, 512), ('dw', 512, 2560, 2816)])
def test_half_width_last_round_single_ctas(which, M, K, N):
    """Without CTA pairs: 220 tiles of 128 x 256 on 148 SMs, 72 in the last round."""
    if sms() != 148:
        pytest.skip('tile counts are chosen for 148 SMs')
    got, expected, schedule = run(which, M, K, N, torch.float16, _lib.FLAG_NO_PAIR)
    assert schedule == 3
    whole, _, _ = run(which, M, K, N, torch.float16, _lib.FLAG_NO_PAIR | _lib.FLAG_WHOLE_TILES)
    assert torch.equal(got, whole)
    torch.testing.assert_close(got.double(), expected, rtol=1e-2, atol=1e-2)


def test_benchmark_weight_gradient_shape():
    """dW of 8192 tokens, 4096 -> 4096: 256 pair tiles = 3 rounds of 74 + 34."""
    if sms() != 148:
        pytest.skip('tile counts are chosen for 148 SMs')
    got, expected, schedule = run('dw', 8192, 4096, 4096, torch.bfloat16, 0)
    assert schedule == 3
    whole, _, _ = run('dw', 8192, 4096, 4096, torch.bfloat16, _lib.FLAG_WHOLE_TILES)
    assert torch.equal(got, whole)


def test_whole_tiles_on_request():
    os.environ['AB200_TAIL_MODE'] = '1'
    _, _, schedule = run('fwd', 2560, 512, 2816, torch.bfloat16, 0)
    assert schedule == 0


@pytest.mark.parametrize('which', ['fwd', 'dx', 'dw'])
def test_full_last_round_as_half_width_units(which):
    """
    148 tiles of 256 x 256 on 74 CTA pairs are two full rounds: whole tiles by default, half-width
    units for the second round with AB200_TAIL_MODE=3.  Ragged variant: the second half of the last
    column block lies beyond N and is skipped.
    """
    if sms() != 148:
        pytest.skip('tile counts are chosen for 148 SMs')
    shape = {'fwd': (9472, 320, 1024), 'dx': (9472, 1024, 320), 'dw': (320, 9472, 1024)}[which]
    whole, expected, schedule = run(which, *shape, torch.bfloat16, 0)
    assert schedule == 0
    os.environ['AB200_TAIL_MODE'] = '3'
    got, _, schedule = run(which, *shape, torch.bfloat16, 0)
    assert schedule == 3
    assert torch.equal(got, whole)
    torch.testing.assert_close(got.double(), expected, rtol=2e-2, atol=2e-2)
    if which == 'fwd':
        got, expected, schedule = run('fwd', 9472, 328, 1024 - 136, torch.bfloat16, 0)
        assert schedule == 3
        whole, _, _ = run('fwd', 9472, 328, 1024 - 136, torch.bfloat16, _lib.FLAG_WHOLE_TILES)
        assert torch.equal(got, whole)
        torch.testing.assert_close(got.double(), expected, rtol=2e-2, atol=2e-2)
