"""
Layer normalisation on the GPU (ab200_layer_norm_forward / ab200_layer_norm_backward behind
attorch_b200.LayerNorm) against the reference's own vectors (tests/golden/layer_norm.npz) and against the
CPU oracle over element types, row widths on both sides of every kernel variant's limits, ragged row
counts and unaligned pitches; then LayerNormLinear against the two layers run one after the other.
The reference's test compares with torch.nn.LayerNorm at rtol = atol = 1e-3
(tests/test_layer_norm_layer.py:56-69); the bounds here are tighter where the arithmetic allows.
"""

import numpy as np
import pytest
import torch

from oracle import linear_oracle as oracle
from tests.helpers import GOLDEN_DIR, LAYER_NORM_BF16_CASES, LAYER_NORM_CASES

pytestmark = pytest.mark.gpu

DTYPES = {'float32': torch.float32, 'float16': torch.float16, 'bfloat16': torch.bfloat16}
# Relative / absolute bounds on values of the given stored type (two ulps of 1 for the 16-bit types; a
# few fp32 ulps times the row length's rounding for fp32).
TOL = {torch.float32: dict(rtol=2e-5, atol=2e-5), torch.float16: dict(rtol=2e-3, atol=2e-3),
       torch.bfloat16: dict(rtol=1.6e-2, atol=1.6e-2)}


def make_layer(feat, eps, affine, bias, dtype, w=None, b=None, autocast_to_fp32=True):
    import attorch_b200
    layer = attorch_b200.LayerNorm(feat, eps, affine, bias, autocast_to_fp32, device='cuda', dtype=dtype)
    with torch.no_grad():
        if affine and w is not None:
            layer.weight.copy_(w)
        if affine and bias and b is not None:
            layer.bias.copy_(b)
    return layer


def run(layer, x, dy, **kwargs):
    xin = x.cuda().requires_grad_(True)
    y = layer(xin, **kwargs)
    y.backward(dy.cuda().to(y.dtype))
    torch.cuda.synchronize()
    dw = layer.weight.grad.cpu() if layer.weight is not None else None
    db = layer.bias.grad.cpu() if layer.bias is not None else None
    return y.detach().cpu(), xin.grad.cpu(), dw, db


def param_grad_tol(dtype, rows, grad):
    # A sum over `rows` terms: a few fp32 ulps of the largest partial sum, plus the rounding to the parameter's type.
    scale = max(1.0, float(grad.abs().max()))
    return dict(rtol=TOL[dtype]['rtol'], atol=TOL[dtype]['atol'] * scale)


@pytest.mark.parametrize('case', range(len(LAYER_NORM_CASES)))
def test_reference_vectors(case):
    shape, dtype_name, affine, bias, eps = LAYER_NORM_CASES[case]
    dtype = DTYPES[dtype_name]
    raw = np.load(GOLDEN_DIR / 'layer_norm.npz')
    g = {k: torch.from_numpy(np.asarray(raw[k])) for k in raw.files if k.endswith(f'_{case}')}
    x, dy = g[f'x_{case}'], g[f'dy_{case}']
    layer = make_layer(shape[-1], eps, affine, bias, dtype, g.get(f'w_{case}'), g.get(f'b_{case}'))
    y, dx, dw, db = run(layer, x, dy)
    assert y.dtype is dtype and dx.dtype is dtype and tuple(y.shape) == shape
    tol = dict(rtol=1e-5, atol=1e-5) if dtype is torch.float32 else dict(rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(y, g[f'y_{case}'], **tol)
    torch.testing.assert_close(dx, g[f'dx_{case}'], **tol)
    if affine:
        rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
        assert dw.dtype is dtype
        torch.testing.assert_close(dw, g[f'dw_{case}'], **param_grad_tol(dtype, rows, g[f'dw_{case}']))
        if bias:
            torch.testing.assert_close(db, g[f'db_{case}'], **param_grad_tol(dtype, rows, g[f'db_{case}']))


# (rows, feat): one warp per row (feat <= 512, rows not a multiple of the 8 rows per block), 256 threads
# per row with and without 16-byte accesses, 512 threads, and rows wider than the registers hold (the
# tail is re-read and the parameter gradients come from the column kernel), aligned and not.
SHAPES = [(1, 1), (3, 7), (37, 64), (1001, 24), (13, 512), (9, 520), (5, 1100), (300, 1024), (6, 4096),
          (700, 4096), (4, 4100), (5, 8192), (3, 8200), (5, 9001), (4, 16384), (600, 12288)]


@pytest.mark.parametrize('dtype', [torch.float32, torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize('rows,feat', SHAPES)
def test_against_oracle(rows, feat, dtype):
    gen = torch.Generator().manual_seed(rows * 131 + feat)
    x = torch.randn(rows, feat, generator=gen) * (torch.rand(rows, 1, generator=gen) * 3 + 0.2) \
        + torch.randn(rows, 1, generator=gen) * 2
    x = x.to(dtype)
    dy = torch.randn(rows, feat, generator=gen).to(dtype)
    w = torch.randn(feat, generator=gen).to(dtype)
    b = torch.randn(feat, generator=gen).to(dtype)
    layer = make_layer(feat, 1e-5, True, True, dtype, w, b)
    y, dx, dw, db = run(layer, x, dy)
    ey, mean, inv_std = oracle.layer_norm_forward(x, w, b, 1e-5)
    edx, edw, edb = oracle.layer_norm_backward(dy, x, mean, inv_std, w, True)
    assert y.dtype is dtype and dx.dtype is dtype
    torch.testing.assert_close(y, ey, **TOL[dtype])
    # dx has cancellation (g minus its projections): bound by the magnitude of the terms, not of the result.
    scale = max(1.0, float((inv_std.max() * (w.float().abs().max() * dy.float().abs().max()))))
    torch.testing.assert_close(dx.float(), edx.float(), rtol=TOL[dtype]['rtol'], atol=TOL[dtype]['atol'] * scale)
    torch.testing.assert_close(dw.float(), edw.to(dtype).float(), **param_grad_tol(dtype, rows, edw))
    torch.testing.assert_close(db.float(), edb.to(dtype).float(), **param_grad_tol(dtype, rows, edb))


@pytest.mark.parametrize('affine,bias', [(False, False), (True, False)])
@pytest.mark.parametrize('rows,feat', [(19, 48), (33, 2048), (7, 10000)])
def test_without_affine_parts(rows, feat, affine, bias):
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(rows, feat, generator=gen) + 1
    dy = torch.randn(rows, feat, generator=gen)
    w = torch.randn(feat, generator=gen) if affine else None
    layer = make_layer(feat, 1e-6, affine, bias, torch.float32, w)
    y, dx, dw, db = run(layer, x, dy)
    ey, mean, inv_std = oracle.layer_norm_forward(x, w, None, 1e-6)
    edx, edw, _ = oracle.layer_norm_backward(dy, x, mean, inv_std, w, False)
    torch.testing.assert_close(y, ey, **TOL[torch.float32])
    torch.testing.assert_close(dx, edx, rtol=2e-5, atol=1e-4)
    assert db is None
    if affine:
        torch.testing.assert_close(dw, edw, **param_grad_tol(torch.float32, rows, edw))
    else:
        assert dw is None


def test_shapes_strides_and_statistics():
    """1-D and 4-D inputs, a strided view, an expanded upstream gradient, and no gradient at all."""
    import attorch_b200
    gen = torch.Generator().manual_seed(11)
    layer = make_layer(40, 1e-5, True, True, torch.float32, torch.randn(40, generator=gen),
                       torch.randn(40, generator=gen))
    w, b = layer.weight.detach().cpu(), layer.bias.detach().cpu()
    for shape in [(40,), (2, 3, 4, 40), (0, 40)]:
        x = torch.randn(shape, generator=gen)
        y = layer(x.cuda())
        assert y.shape == x.shape
        torch.testing.assert_close(y.detach().cpu(), oracle.layer_norm_forward(x, w, b)[0], **TOL[torch.float32])
    tall = torch.randn(6, 10, 80, generator=gen)
    view = tall[:, ::2, 20:60]                           # rows of 40 at a pitch of 160 elements
    xin = tall.cuda()[:, ::2, 20:60].detach().requires_grad_(True)
    assert xin.stride() == (800, 160, 1)
    layer.zero_grad()
    y = layer(xin)
    y.sum().backward()                                   # the engine hands backward an expanded tensor of ones
    ey, mean, inv_std = oracle.layer_norm_forward(view.contiguous(), w, b)
    edx, edw, edb = oracle.layer_norm_backward(torch.ones_like(ey), view.contiguous(), mean, inv_std, w, True)
    torch.testing.assert_close(y.detach().cpu(), ey, **TOL[torch.float32])
    torch.testing.assert_close(xin.grad.cpu(), edx, rtol=2e-5, atol=1e-4)
    torch.testing.assert_close(layer.weight.grad.cpu(), edw, rtol=2e-5, atol=1e-4)
    torch.testing.assert_close(layer.bias.grad.cpu(), edb, rtol=2e-5, atol=1e-4)
    # A row start that is not 16-byte aligned, on a width the 16-byte variant would otherwise take.
    wide = torch.randn(5, 4100, generator=gen)
    plain = make_layer(4096, 1e-5, False, False, torch.float32)
    torch.testing.assert_close(plain(wide.cuda()[:, 1:4097]).cpu(),
                               oracle.layer_norm_forward(wide[:, 1:4097].contiguous())[0], **TOL[torch.float32])
    # Parameters frozen, input needs a gradient: only dx comes back.
    frozen = make_layer(40, 1e-5, True, True, torch.float32, w, b)
    frozen.requires_grad_(False)
    xin = tall[0].contiguous()[:, :40].cuda().requires_grad_(True)
    frozen(xin).sum().backward()
    assert xin.grad is not None and frozen.weight.grad is None
    attorch_b200.check_status()


@pytest.mark.parametrize('input_dtype', [torch.float32, torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize('autocast_dtype', [torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize('to_fp32', [True, False])
def test_autocast_rule(input_dtype, autocast_dtype, to_fp32):
    """
    Under autocast the output is fp32, or the input's dtype with autocast_to_fp32 off (attorch/
    layer_norm_layer.py:55-56); parameters stay fp32; gradients reach the leaves in their own dtypes.
    """
    gen = torch.Generator().manual_seed(3)
    x = (torch.randn(4, 9, 1024, generator=gen) * 2 + 0.5).to(input_dtype)
    dy = torch.randn(4, 9, 1024, generator=gen)
    w, b = torch.randn(1024, generator=gen), torch.randn(1024, generator=gen)
    layer = make_layer(1024, 1e-5, True, True, torch.float32, w, b, autocast_to_fp32=to_fp32)
    xin = x.cuda().requires_grad_(True)
    with torch.autocast('cuda', dtype=autocast_dtype):
        y = layer(xin)
    expected_dtype = torch.float32 if to_fp32 else input_dtype
    assert y.dtype is expected_dtype
    y.backward(dy.cuda().to(y.dtype))
    assert xin.grad.dtype is input_dtype and layer.weight.grad.dtype is torch.float32
    ey, mean, inv_std = oracle.layer_norm_forward(x, w, b, output_dtype=expected_dtype)
    edx, edw, edb = oracle.layer_norm_backward(dy.to(expected_dtype), x, mean, inv_std, w, True, grad_dtype=expected_dtype)
    torch.testing.assert_close(y.detach().cpu(), ey, **TOL[expected_dtype])
    torch.testing.assert_close(xin.grad.cpu().float(), edx.to(input_dtype).float(), rtol=TOL[input_dtype]['rtol'],
                               atol=TOL[input_dtype]['atol'] * 8)
    # Both sides see the same rounded dy and add in fp32: only the order of the additions differs.
    torch.testing.assert_close(layer.weight.grad.cpu(), edw, rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(layer.bias.grad.cpu(), edb, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize('autocast_dtype', [torch.float16, torch.bfloat16], ids=str)
# More than 128 tokens: below that the projection adds split reductions with atomics, whose order varies from run to run.
@pytest.mark.parametrize('tokens,dim,hidden', [(200, 256, 512), (520, 1024, 768)])
def test_layer_norm_linear_equals_the_two_layers(tokens, dim, hidden, autocast_dtype):
    """
    LayerNormLinear under autocast against LayerNorm followed by Linear: the projection sees the same
    operand bits, so outputs are bit-equal; the gradients differ only in that the fused path rounds the
    projection's input gradient to the autocast dtype (as the reference does, attorch/linear_layer.py:
    152-153) where this package's Linear alone writes it in fp32 unrounded.
    """
    import attorch_b200
    gen = torch.Generator().manual_seed(17)
    x = torch.randn(tokens, dim, generator=gen) * 1.5 + 0.3
    dy = torch.randn(tokens, hidden, generator=gen) * 0.05
    torch.manual_seed(0)
    norm = attorch_b200.LayerNorm(dim)
    linear = attorch_b200.Linear(dim, hidden, act_func='gelu')
    with torch.no_grad():
        norm.weight.copy_(torch.randn(dim, generator=gen))
        norm.bias.copy_(torch.randn(dim, generator=gen))
    fused = attorch_b200.LayerNormLinear(norm, linear)

    def step(module_call):
        for p in fused.parameters():
            p.grad = None
        xin = x.cuda().requires_grad_(True)
        with torch.autocast('cuda', dtype=autocast_dtype):
            y = module_call(xin)
        y.backward(dy.cuda().to(y.dtype))
        torch.cuda.synchronize()
        return [y.detach().cpu(), xin.grad.cpu()] + [p.grad.cpu().clone() for p in fused.parameters()]

    got = step(fused)
    want = step(lambda t: linear(norm(t)))
    assert got[0].dtype is autocast_dtype and got[1].dtype is torch.float32
    assert torch.equal(got[0], want[0])
    names = ['dx', 'norm.weight', 'norm.bias', 'linear.weight', 'linear.bias']
    for name, a, b in zip(names, got[1:], want[1:]):
        if name.startswith('linear'):
            assert torch.equal(a, b), name          # same operands, same kernels
        else:
            scale = max(1.0, float(b.abs().max()))
            torch.testing.assert_close(a, b, rtol=TOL[autocast_dtype]['rtol'], atol=TOL[autocast_dtype]['atol'] * scale,
                                       msg=lambda m: f'{name}: {m}')
    # And against the oracle chain: normalisation output rounded to the operand dtype.
    w, b = norm.weight.detach().cpu(), norm.bias.detach().cpu()
    operand = oracle.layer_norm_forward(x, w, b, output_dtype=autocast_dtype)[0]
    with torch.autocast('cuda', dtype=autocast_dtype):
        y_direct = linear(operand.cuda())
    # The CPU sums rows in another order: a few operand elements land on the other side of a rounding boundary.
    torch.testing.assert_close(y_direct.cpu().float(), got[0].float(), rtol=TOL[autocast_dtype]['rtol'],
                               atol=TOL[autocast_dtype]['atol'])
    attorch_b200.check_status()


def test_c_abi_argument_checks():
    """Rejected calls return a negative code and launch nothing."""
    from attorch_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(4, 64, device='cuda')
    y = torch.zeros(4, 64, device='cuda', dtype=torch.float16)
    stats = torch.zeros(2, 4, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    before = lib.ab200_launch_count()
    call = lib.ab200_layer_norm_forward
    assert call(x.data_ptr(), None, None, stats[0].data_ptr(), stats[1].data_ptr(), y.data_ptr(), 4, 0, 64, 64,
                _lib.F32, 0, _lib.F16, 1e-5, stream) == -2                         # no features
    assert call(x.data_ptr(), None, None, stats[0].data_ptr(), None, y.data_ptr(), 4, 64, 64, 64,
                _lib.F32, 0, _lib.F16, 1e-5, stream) == -1                         # one statistic only
    assert call(x.data_ptr(), None, x.data_ptr(), None, None, y.data_ptr(), 4, 64, 64, 64,
                _lib.F32, 0, _lib.F16, 1e-5, stream) == -1                         # bias without weight
    assert call(y.data_ptr(), None, None, None, None, y.data_ptr(), 4, 64, 64, 64,
                _lib.BF16, 0, _lib.F16, 1e-5, stream) == -3                        # bf16 -> fp16
    assert call(x.data_ptr(), None, None, None, None, y.data_ptr(), 4, 64, 32, 64,
                _lib.F32, 0, _lib.F16, 1e-5, stream) == -5                         # pitch below the row length
    back = lib.ab200_layer_norm_backward
    assert back(x.data_ptr(), x.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(), x.data_ptr(), x.data_ptr(),
                x.data_ptr(), None, 4, 64, 64, 64, 64, _lib.F32, _lib.F32, _lib.F32, _lib.F32, x.data_ptr(), 16,
                None, stream) == -6                                                      # workspace too small
    assert back(x.data_ptr(), x.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(), x.data_ptr(), x.data_ptr(),
                None, None, 4, 64, 64, 64, 64, _lib.F16, _lib.F32, _lib.F32, _lib.F16, None, 0,
                None, stream) == -3                                                      # dx narrower than x
    assert lib.ab200_launch_count() == before
    assert lib.ab200_layer_norm_workspace_bytes(0, 64) == 4
    assert lib.ab200_layer_norm_workspace_bytes(8192, 4096) % (2 * 4096 * 4) == 0


@pytest.mark.parametrize('rows,feat', [(300, 1024), (150, 4096), (40, 8192)])
@pytest.mark.parametrize('x_dtype,dy_dtype', [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                              (torch.bfloat16, torch.bfloat16), (torch.float16, torch.float32)],
                         ids=['f32', 'f32_bf16', 'bf16', 'f16_f32'])
def test_staged_and_register_backward_agree(rows, feat, x_dtype, dy_dtype):
    """
    The backward pass with rows staged in shared memory (a status word is given) and the one that keeps
    rows in registers (no status word) do the same arithmetic with different thread-to-column maps: equal
    up to the order of the row sums.  Both against the oracle.
    """
    from attorch_b200 import _lib
    lib = _lib.load()
    ids = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
    gen = torch.Generator().manual_seed(rows + feat)
    x = (torch.randn(rows, feat, generator=gen) * 2 + 0.7).to(x_dtype)
    dy = torch.randn(rows, feat, generator=gen).to(dy_dtype)
    w = torch.randn(feat, generator=gen)
    dx_dtype = torch.float32 if torch.float32 in (x_dtype, dy_dtype) else x_dtype
    _, mean, inv_std = oracle.layer_norm_forward(x, w, None)
    edx, edw, edb = oracle.layer_norm_backward(dy, x, mean, inv_std, w, True, grad_dtype=dx_dtype)
    xg, dyg, wg, stats = x.cuda(), dy.cuda(), w.cuda(), torch.stack([mean, inv_std]).cuda()
    ws = torch.empty(lib.ab200_layer_norm_workspace_bytes(rows, feat), dtype=torch.uint8, device='cuda')
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for status_ptr in (status.data_ptr(), None):
        dx = torch.empty(rows, feat, dtype=dx_dtype, device='cuda')
        pg = torch.empty(2, feat, device='cuda')
        _lib.check(lib.ab200_layer_norm_backward(
            dyg.data_ptr(), xg.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(), wg.data_ptr(), dx.data_ptr(),
            pg[0].data_ptr(), pg[1].data_ptr(), rows, feat, feat, feat, feat, ids[dy_dtype], ids[x_dtype], _lib.F32,
            ids[dx_dtype], ws.data_ptr(), ws.numel(), status_ptr, stream), 'ab200_layer_norm_backward')
        torch.cuda.synchronize()
        outs.append((dx.cpu(), pg[0].cpu(), pg[1].cpu()))
    assert int(status.item()) == 0
    scale = max(1.0, float(inv_std.max() * w.abs().max() * dy.float().abs().max()))
    for dx, dw, db in outs:
        torch.testing.assert_close(dx.float(), edx.float(), rtol=TOL[dx_dtype]['rtol'], atol=TOL[dx_dtype]['atol'] * scale)
        torch.testing.assert_close(dw, edw, rtol=1e-4, atol=1e-4 * max(1.0, float(edw.abs().max())))
        torch.testing.assert_close(db, edb, rtol=1e-4, atol=1e-4 * max(1.0, float(edb.abs().max())))
    torch.testing.assert_close(outs[0][0].float(), outs[1][0].float(), rtol=TOL[dx_dtype]['rtol'],
                               atol=TOL[dx_dtype]['atol'] * scale)


@pytest.mark.parametrize('case', range(len(LAYER_NORM_BF16_CASES)))
def test_reference_bf16_vectors(case):
    """
    Against the reference's own bf16 runs (tests/golden/layer_norm_bf16.npz).  The interpreter that made them
    stores fp32 values as bf16 by truncation, a GPU rounds to nearest: the kernel's value is the vector's or
    the next bf16 number away from zero, never more than one step off.
    """
    shape, param_dtype_name, bias = LAYER_NORM_BF16_CASES[case]
    raw = np.load(GOLDEN_DIR / 'layer_norm_bf16.npz')
    g = {k: torch.from_numpy(np.asarray(raw[k])) for k in raw.files if k.endswith(f'_{case}')}
    param_dtype = DTYPES[param_dtype_name]
    layer = make_layer(shape[-1], 1e-5, True, bias, param_dtype, g[f'w_{case}'], g.get(f'b_{case}'))
    y, dx, dw, db = run(layer, g[f'x_{case}'].bfloat16(), g[f'dy_{case}'].bfloat16())
    assert y.dtype is torch.bfloat16 and dx.dtype is torch.bfloat16 and dw.dtype is param_dtype
    for name, got, ref in (('y', y.float(), g[f'y_{case}']), ('dx', dx.float(), g[f'dx_{case}'])):
        step = torch.maximum(ref.abs(), torch.tensor(1e-30)) * 2.0 ** -7
        assert bool(((got - ref).abs() <= step).all()), name
        away = (got.abs() >= ref.abs()) | ((got - ref).abs() <= step * 1e-3)
        assert away.float().mean() >= 0.98, name      # rounding to nearest never lands below a truncated value
    scale = max(1.0, float(g[f'dw_{case}'].abs().max()))
    tol = dict(rtol=1e-4, atol=1e-4 * scale) if param_dtype is torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2 * scale)
    torch.testing.assert_close(dw.float(), g[f'dw_{case}'], **tol)
    if bias:
        torch.testing.assert_close(db.float(), g[f'db_{case}'], **tol)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16], ids=str)
def test_full_size_properties(dtype):
    """
    The bench's shape, 8192 rows of 4096 features, through properties that need no CPU product: normalised
    rows have mean 0 and mean square var / (var + eps); each row of dx sums to 0; a sample of rows of dx equals
    the formula evaluated in float64; dw and db equal float64 column sums taken from the layer's own normalised
    output; backward is linear in the upstream gradient.
    """
    import attorch_b200
    rows, feat = 8192, 4096
    gen = torch.Generator(device='cuda').manual_seed(1)
    x = (torch.randn(rows, feat, device='cuda', generator=gen) * (torch.rand(rows, 1, device='cuda', generator=gen) * 3 + 0.2)
         + torch.randn(rows, 1, device='cuda', generator=gen) * 2).to(dtype)
    dy1 = torch.randn(rows, feat, device='cuda', generator=gen).to(dtype)
    dy2 = torch.randn(rows, feat, device='cuda', generator=gen).to(dtype)
    w = torch.randn(feat, device='cuda', generator=gen).to(dtype)
    unit = 2.0 ** -8 if dtype is torch.bfloat16 else 2.0 ** -22          # about one rounding of a value near 1

    plain = attorch_b200.LayerNorm(feat, elementwise_affine=False, dtype=dtype)
    xin = x.clone().requires_grad_(True)
    p = plain(xin)
    p64 = p.detach().double()
    x64 = x.double()
    mu, var = x64.mean(dim=1), x64.var(dim=1, unbiased=False)
    # A row far from zero loses |mean| / std of the fp32 resolution in (x - mean); mean square is var / (var + eps).
    slack = 32 * unit * (1 + mu.abs() / var.sqrt())
    assert bool((p64.mean(dim=1).abs() <= slack).all())
    assert bool(((p64.pow(2).mean(dim=1) - var / (var + 1e-5)).abs() <= 2 * slack).all())

    layer = attorch_b200.LayerNorm(feat, dtype=dtype)
    with torch.no_grad():
        layer.weight.copy_(w)

    def backward(dy):
        layer.zero_grad()
        xg = x.clone().requires_grad_(True)
        layer(xg).backward(dy)
        return xg.grad.double(), layer.weight.grad.double(), layer.bias.grad.double()

    dx1, dw1, db1 = backward(dy1)
    g = (w.double() * dy1.double())
    rs = 1.0 / (var + 1e-5).sqrt()
    row_scale = rs * g.abs().max(dim=1).values                         # magnitude of the terms of a row of dx
    scale = float(row_scale.max())
    # Each row of dx sums to zero (the mean of g and its projection on the normalised row are taken out).
    assert bool((dx1.sum(dim=1).abs() <= (1e-3 if dtype is torch.float32 else 0.3) * row_scale).all())
    # A sample of rows against the formula in float64.
    idx = torch.arange(0, rows, 127, device='cuda')
    ps, gs = ((x64[idx] - mu[idx, None]) * rs[idx, None]), g[idx]
    ref_dx = rs[idx, None] * (gs - (ps * (ps * gs).mean(dim=1, keepdim=True) + gs.mean(dim=1, keepdim=True)))
    assert bool(((dx1[idx] - ref_dx).abs() <= 16 * unit * row_scale[idx, None] + 1e-6).all())
    # Parameter gradients against float64 sums over the rows (p from the layer's own forward: one rounding off).
    ref_dw = (dy1.double() * p64).sum(dim=0)
    ref_db = dy1.double().sum(dim=0)
    col = float((dy1.double().abs() * p64.abs()).sum(dim=0).max())
    assert float((dw1 - ref_dw).abs().max()) <= 4 * unit * col
    assert float((db1 - ref_db).abs().max()) <= 4 * unit * float(dy1.double().abs().sum(dim=0).max())
    # Linearity in the upstream gradient.
    dx2, dw2, _ = backward(dy2)
    dx12, dw12, _ = backward((dy1.float() * 0.5 + dy2.float()).to(dtype))
    assert float((dx12 - (0.5 * dx1 + dx2)).abs().max()) <= 128 * unit * scale
    assert float((dw12 - (0.5 * dw1 + dw2)).abs().max()) <= 16 * unit * col
    attorch_b200.check_status()
