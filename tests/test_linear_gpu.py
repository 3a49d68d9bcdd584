"""
GPU parity tests of the fused linear layer: the CUDA kernels, called through the C ABI by
attorch_b200.Linear, against (1) golden vectors produced by the reference itself and (2) the CPU
oracle on seeded inputs.  Tolerance: rtol = atol = 1e-2 for bf16 / fp16 / TF32 (fp32 accumulation),
1e-4 where the exact-fp32 generic kernel is forced; shapes and dtypes must match exactly.

Backward differentiates through the STORED pre-activation (attorch/linear_layer.py:104-105,
143-146 of the reference).  Two correct forward passes can round a pre-activation that lies within
one rounding error of a kink of the activation (0 for relu, +-lambda for the shrinks, ...) to
opposite sides of it, which flips that element's derivative between 0 and 1.  The gradient checks
therefore feed the oracle's backward the pre-activation the GPU stored (obtained from the same
kernel with the activation switched off, which is bit-identical), while the forward output is
checked against the oracle's own forward.  On the exact-fp32 generic kernel no such flip can
happen and everything is compared with the reference's golden vectors directly.

Where the CUDA path deliberately differs from the reference the oracle is asked for the same
arithmetic, so that the comparison stays tight:
  * fp32 operands are multiplied as TF32 in all three products on the tcgen05 kernels (the
    reference: TF32 in forward, true fp32 in its cuBLAS backward).  The tensor cores truncate fp32
    operands to TF32 (test_tf32_operands_are_truncated pins that), so the oracle truncates too.
  * Activation derivatives are evaluated in fp32 for every activation; the reference evaluates
    the piecewise ones in the 16-bit dtype of the stored pre-activation, whose per-operation
    rounding is looser than this comparison's tolerance.
  * Gradients of fp32 parameters / inputs under 16-bit autocast are written from the fp32
    accumulator without an intermediate rounding to the autocast dtype.
"""

import pytest
import torch

import attorch_b200
from attorch_b200 import _lib
from oracle import linear_oracle as oracle
from tests.helpers import assert_close, golden_names, load_golden

pytestmark = pytest.mark.gpu

DEV = 'cuda'
TOL = 1e-2


def make_layer(w, b, act_func, dtype):
    layer = attorch_b200.Linear(w.shape[0], w.shape[1], bias=b is not None, act_func=act_func,
                                device=DEV, dtype=dtype)
    with torch.no_grad():
        layer.weight.copy_(w)
        if b is not None:
            layer.bias.copy_(b)
    return layer


LAST_PATH = {'path': None}
SAVE_DERIVATIVE = {'on': True}      # the layer's default: forward saves act'(Z)
SAVED = {'tensor': None}


def run_layer(x, w, b, act_func, dy, autocast_dtype=None, flags=0, param_dtype=None):
    """
    Forward + backward on the GPU.  Returns (y, dx, dw, db, z): the results on the CPU and the
    pre-activation the kernel stored (None without an activation).  LAST_PATH['path'] records
    which kernel family the forward call used.
    """
    layer = make_layer(w, b, act_func, param_dtype or w.dtype)
    xg = x.to(DEV).requires_grad_(True)
    previous = attorch_b200.set_gemm_flags(flags)
    try:
        with torch.autocast('cuda', dtype=autocast_dtype or torch.float16,
                            enabled=autocast_dtype is not None):
            y = layer(xg)
            LAST_PATH['path'] = _lib.load().ab200_last_path()
            # What forward kept for backward: Z, or act'(Z) in the default save-derivative mode.
            SAVED['tensor'] = y.grad_fn.saved_tensors[1].cpu() if act_func is not None else None
            z = None
            if act_func is not None:
                with torch.no_grad():
                    z = make_layer(w, b, None, param_dtype or w.dtype)(xg.detach()).cpu()
        y.backward(dy.to(DEV).to(y.dtype))
        attorch_b200.check_status()
    finally:
        attorch_b200.set_gemm_flags(previous)
    db = layer.bias.grad.cpu() if b is not None else None
    return y.detach().cpu(), xg.grad.cpu(), layer.weight.grad.cpu(), db, z


def expected_from_oracle(x, w, b, act_func, dy, z_gpu, autocast_dtype=None):
    """Oracle forward, and oracle backward through the pre-activation the GPU stored."""
    out_dtype = oracle.output_dtype_rule(x.dtype, autocast_dtype)
    tensor_cores = LAST_PATH['path'] != _lib.PATH_GENERIC
    tf32 = 'truncate' if (out_dtype is torch.float32 and tensor_cores) else None
    y, z = oracle.linear_forward(x, w, b, act_func, autocast_dtype, tf32=tf32)
    if z_gpu is not None:
        assert_close(z_gpu.view_as(z), z, TOL, 'pre-activation')
        z = z_gpu.view_as(z)
    name, param = oracle.parse_act_func(act_func)
    stored = None
    if name is not None and SAVE_DERIVATIVE['on']:
        # The saved derivative against the oracle's act'(stored Z), then backward through it: two
        # correct evaluations can round act'(Z) to neighbouring 16-bit values, and backward reads
        # the stored one.
        stored = SAVED['tensor'].view_as(z)
        # (A bf16 layer keeps it as fp16: same size, finer spacing.)
        assert stored.dtype is (torch.float16 if out_dtype is torch.bfloat16 else out_dtype)
        assert_close(stored, oracle.act_grad(name, z.float(), param).to(stored.dtype), TOL, 'saved derivative')
    dx, dw, db = oracle.linear_backward(dy.to(out_dtype), x, z, w, act_func, out_dtype, b, tf32=tf32,
                                        derivative_in_fp32=True, round_to_out_dtype=False,
                                        stored_derivative=stored)
    if b is not None:
        # db: fp32 sum of the stored dZ, rounded once to the bias dtype.
        dz = dy.to(out_dtype).flatten(0, -2)
        if stored is not None:
            dz = (dz.float() * stored.float()).to(out_dtype)
        elif name is not None:
            dz = (dz * oracle.act_grad(name, z.float(), param)).to(out_dtype)
        db = dz.float().sum(0).to(b.dtype)
    return y, dx, dw, db


def test_tf32_operands_are_truncated():
    """fp32 operands reach the tensor cores as TF32 by dropping the low 13 mantissa bits."""
    values = [1 + 3 * 2 ** -12, 1 + 2 ** -11, 1 + 2 ** -12, 1 + 2 ** -10 + 2 ** -11, -(1 + 3 * 2 ** -12)]
    x = torch.zeros(256, 32)
    x[:len(values), 0] = torch.tensor(values)
    w = torch.zeros(32, 64)
    w[0, 0] = 1.0
    layer = make_layer(w, None, None, torch.float32)
    previous = attorch_b200.set_gemm_flags(_lib.FLAG_FORCE_TCGEN05 | _lib.FLAG_NO_STREAMK)
    try:
        with torch.no_grad():
            y = layer(x.to(DEV)).cpu()
    finally:
        attorch_b200.set_gemm_flags(previous)
    attorch_b200.check_status()
    expect = oracle.tf32_round(torch.tensor(values), 'truncate')
    assert torch.equal(y[:len(values), 0], expect)


def check_against(expected, got, tol, has_bias=True):
    names = ('output', 'input grad', 'weight grad', 'bias grad')
    for name, e, g in zip(names, expected, got):
        if name == 'bias grad' and not has_bias:
            assert g is None
            continue
        assert_close(g, e, tol, name)


def check_layer(x, w, b, act_func, dy, tol=TOL, autocast_dtype=None, flags=0):
    got = run_layer(x, w, b, act_func, dy, autocast_dtype=autocast_dtype, flags=flags)
    expected = expected_from_oracle(x, w, b, act_func, dy, got[4], autocast_dtype)
    check_against(expected, got[:4], tol, has_bias=b is not None)
    return got


# ------------------------------------------------------------------------------------------------
# 1. Golden vectors made by the reference
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('name', golden_names())
def test_golden_exact_kernel(name):
    """The exact-fp32 generic kernel reproduces the reference's output and gradients."""
    case = load_golden(name)
    got = run_layer(case['x'], case['w'], case['b'], case['act_func'], case['dy'],
                    flags=_lib.FLAG_FORCE_GENERIC)
    expected = (case['y'], case['dx'], case['dw'], case['db'])
    tol = 1e-4 if case['dtype'] is torch.float32 else TOL
    check_against(expected, got[:4], tol, has_bias=case['b'] is not None)


@pytest.mark.parametrize('name', golden_names())
def test_golden_default_kernels(name):
    """
    Whatever kernels the library picks (tcgen05 where TMA can address the operands): the output
    against the reference's golden output, the gradients through the stored pre-activation.
    """
    case = load_golden(name)
    got = check_layer(case['x'], case['w'], case['b'], case['act_func'], case['dy'])
    assert_close(got[0], case['y'], TOL, 'output vs reference')
    kinked = case['act_func'] is not None and case['act_func'].split('_')[0] not in oracle.FP32_ACTS
    if not kinked or not name.startswith('config1'):
        # Away from derivative flips the reference's own gradients are matched as well.
        if not name.startswith('switch_'):
            assert_close(got[1], case['dx'], TOL, 'input grad vs reference')
            assert_close(got[2], case['dw'], TOL, 'weight grad vs reference')


@pytest.mark.parametrize('name', golden_names('switch_'))
def test_golden_switch_points_exact_on_generic_kernel(name):
    """Exact-fp32 kernel: the piecewise conventions at the switch points are bit-exact."""
    case = load_golden(name)
    act = case['act_func']
    if act is not None and act.split('_')[0] in oracle.FP32_ACTS | {'softsign'}:
        pytest.skip('no switch point')
    got = run_layer(case['x'], case['w'], case['b'], act, case['dy'], flags=_lib.FLAG_FORCE_GENERIC)
    assert torch.equal(got[0], case['y'])
    assert torch.equal(got[1], case['dx'])


# ------------------------------------------------------------------------------------------------
# 2. Seeded inputs against the oracle, per kernel family
# ------------------------------------------------------------------------------------------------
def seeded(shape, out_dim, dtype, seed=0, bias=True, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    x = (torch.randn(shape, generator=gen) * scale).to(dtype)
    w = (torch.randn((shape[-1], out_dim), generator=gen) / shape[-1] ** 0.5).to(dtype)
    b = torch.randn(out_dim, generator=gen).to(dtype) if bias else None
    dy = torch.randn((*shape[:-1], out_dim), generator=gen).to(dtype)
    return x, w, b, dy


SHAPES = [
    ((1536, 320), 768),      # several 256-row tiles (CTA pairs), ragged k-blocks
    ((128, 64), 256),        # exactly one tile, one k-block
    ((256, 512), 512),       # several tiles and k-blocks
    ((300, 264), 520),       # ragged in M, K and N
    ((4, 50, 128), 96),      # 3-D input, narrow N
    ((1000, 72), 40),        # short K, N below one MMA atom width of 64
    ((129, 2048), 136),      # long K
]
FAMILIES = [('tcgen05', _lib.FLAG_FORCE_TCGEN05 | _lib.FLAG_NO_STREAMK),
            ('tcgen05-1cta', _lib.FLAG_FORCE_TCGEN05 | _lib.FLAG_NO_STREAMK | _lib.FLAG_NO_PAIR),
            ('tcgen05-regstore', _lib.FLAG_FORCE_TCGEN05 | _lib.FLAG_NO_STREAMK | _lib.FLAG_NO_TMA_STORE),
            ('streamk', _lib.FLAG_FORCE_TCGEN05 | _lib.FLAG_FORCE_STREAMK),
            ('generic', _lib.FLAG_FORCE_GENERIC)]


@pytest.mark.parametrize('family,flags', FAMILIES)
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('shape,out_dim', SHAPES)
@pytest.mark.parametrize('act_func', [None, 'gelu', 'relu'])
def test_oracle_parity(family, flags, dtype, shape, out_dim, act_func):
    x, w, b, dy = seeded(shape, out_dim, dtype)
    # Exact fp32 products on the generic kernel; what is left is fp32 summation order.
    tol = 5e-4 if (family == 'generic' and dtype is torch.float32) else TOL
    check_layer(x, w, b, act_func, dy, tol=tol, flags=flags)


@pytest.mark.parametrize('act_func', oracle.ALL_ACT_FUNCS)
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('save_derivative', [True, False])
def test_every_activation(act_func, dtype, save_derivative):
    """Every activation, with forward saving act'(Z) (default) and saving Z as the reference does."""
    x, w, b, dy = seeded((200, 192), 320, dtype, seed=3)
    previous = attorch_b200.set_save_derivative(save_derivative)
    SAVE_DERIVATIVE['on'] = save_derivative
    try:
        check_layer(x, w, b, act_func, dy)
    finally:
        attorch_b200.set_save_derivative(previous)
        SAVE_DERIVATIVE['on'] = True


@pytest.mark.parametrize('autocast_dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('input_dtype', [torch.float32, torch.float16])
def test_autocast(autocast_dtype, input_dtype):
    """fp32 parameters under autocast: 16-bit output, gradients in the parameters' dtypes."""
    x, w, b, dy = seeded((6, 40, 256), 384, torch.float32, seed=5)
    x = x.to(input_dtype)
    got = check_layer(x, w, b, 'silu', dy, autocast_dtype=autocast_dtype)
    assert got[0].dtype is autocast_dtype
    assert got[1].dtype is input_dtype and got[2].dtype is torch.float32 and got[3].dtype is torch.float32


# ------------------------------------------------------------------------------------------------
# 3. Edge cases of the drop-in contract
# ------------------------------------------------------------------------------------------------
def test_strided_input_and_expanded_grad():
    """Non-contiguous input; y.sum().backward() hands backward a zero-stride gradient."""
    torch.manual_seed(0)
    tall = torch.randn(8, 20, 64)
    x = tall[:, ::2, :]
    w = torch.randn(64, 48) / 8
    b = torch.randn(48)
    layer = make_layer(w, b, 'tanh', torch.float32)
    xg = x.to(DEV).requires_grad_(True)
    y = layer(xg)
    y.sum().backward()
    attorch_b200.check_status()
    e_y, _, e_dx, e_dw, e_db = oracle.linear_forward_backward(x, w, b, 'tanh', torch.ones(8, 10, 48))
    check_against((e_y, e_dx, e_dw, e_db),
                  (y.detach().cpu(), xg.grad.cpu(), layer.weight.grad.cpu(), layer.bias.grad.cpu()), TOL)


@pytest.mark.parametrize('shape,out_dim', [((1, 8000), 16), ((12288, 1), 16), ((5, 196), 196),
                                           ((2048, 64, 16), 96), ((3, 7), 1)])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float16])
def test_reference_test_matrix_odd_shapes(shape, out_dim, dtype):
    """Shapes from the reference's own test matrix that TMA cannot address or that are tiny."""
    x, w, b, dy = seeded(shape, out_dim, dtype, seed=7)
    check_layer(x, w, b, 'relu', dy)


def test_empty_batch():
    layer = attorch_b200.Linear(32, 48, act_func='relu', device=DEV)
    x = torch.empty(0, 32, device=DEV, requires_grad=True)
    y = layer(x)
    assert y.shape == (0, 48)
    y.sum().backward()
    attorch_b200.check_status()
    assert x.grad.shape == (0, 32)
    assert torch.count_nonzero(layer.weight.grad) == 0 and torch.count_nonzero(layer.bias.grad) == 0


def test_requires_grad_combinations():
    x, w, b, dy = seeded((64, 128), 128, torch.float32, seed=9)
    layer = make_layer(w, b, 'gelu', torch.float32)
    # Input without grad: only parameter gradients.
    y = layer(x.to(DEV))
    y.backward(dy.to(DEV))
    assert layer.weight.grad is not None and layer.bias.grad is not None
    # Frozen parameters: only the input gradient.
    frozen = make_layer(w, b, 'gelu', torch.float32)
    for p in frozen.parameters():
        p.requires_grad_(False)
    xg = x.to(DEV).requires_grad_(True)
    frozen(xg).backward(dy.to(DEV))
    assert xg.grad is not None and frozen.weight.grad is None and frozen.bias.grad is None
    # no_grad forward.
    with torch.no_grad():
        y2 = layer(x.to(DEV))
    assert not y2.requires_grad
    attorch_b200.check_status()
    torch.testing.assert_close(y2, y.detach())


def test_error_behaviour():
    layer = attorch_b200.Linear(16, 8, device=DEV)
    with pytest.raises(AssertionError, match='Incompatible input'):
        layer(torch.randn(4, 15, device=DEV))
    with pytest.raises(IndexError):
        layer(torch.randn(16, device=DEV))
    with pytest.raises(ValueError):
        attorch_b200.Linear(16, 8, act_func='leaky_relu', device=DEV)(torch.randn(2, 16, device=DEV))
    with pytest.raises(ValueError):
        attorch_b200.Linear(16, 8, act_func='swish', device=DEV)(torch.randn(2, 16, device=DEV))
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        attorch_b200.Linear(16, 8, device='cpu')(torch.randn(2, 16))


def test_state_dict_layout():
    layer = attorch_b200.Linear(24, 40, device=DEV)
    sd = layer.state_dict()
    assert sd['weight'].shape == (24, 40) and sd['bias'].shape == (40,)
    assert layer.in_features == 24 and layer.out_features == 40


def test_bitwise_repeatable():
    """Same inputs, same bits: catches pipeline races in the warp-specialised kernels."""
    x, w, b, dy = seeded((1024, 1024), 1024, torch.bfloat16, seed=11)
    first = run_layer(x, w, b, 'gelu', dy)
    for _ in range(5):
        again = run_layer(x, w, b, 'gelu', dy)
        for a, c in zip(first, again):
            assert torch.equal(a, c)


# ------------------------------------------------------------------------------------------------
# 4. Full-size benchmark configurations, checked through sub-sampled oracle products
# ------------------------------------------------------------------------------------------------
def test_config2_full_size_bf16():
    """
    The headline configuration (bf16, M = 8192, 4096 -> 4096, gelu, bias).  The oracle is evaluated on 48
    sampled rows (output, dX) and 48 sampled input features (dW); db in full.
    """
    torch.manual_seed(0)
    M, K, N = 8192, 4096, 4096
    x = torch.randn(M, K).bfloat16()
    lin = torch.nn.Linear(K, N)
    w = lin.weight.detach().T.contiguous().bfloat16()
    b = lin.bias.detach().bfloat16()
    dy = (torch.randn(M, N) * 0.01).bfloat16()
    y, dx, dw, db, z = run_layer(x, w, b, 'gelu', dy)
    rows = torch.randperm(M)[:48]
    e_y, e_z = oracle.linear_forward(x[rows], w, b, 'gelu')
    assert_close(y[rows], e_y, TOL, 'output rows')
    assert_close(z[rows], e_z, TOL, 'pre-activation rows')
    e_dx, _, _ = oracle.linear_backward(dy[rows], x[rows], z[rows], w, 'gelu', torch.bfloat16, b,
                                        derivative_rounded=True)
    assert_close(dx[rows], e_dx, TOL, 'dX rows')
    # dW and db sum over all 8192 rows.  With dZ from the oracle's activation backward on the full
    # stored pre-activation (elementwise, cheap), 48 sampled input features of dW and all of db are
    # checked with float64 products.
    dz = (dy.float() * oracle.act_grad('gelu', z.float()).bfloat16().float()).bfloat16()
    feats = torch.randperm(K)[:48]
    e_dw = (x[:, feats].double().T @ dz.double()).float().bfloat16()
    assert_close(dw[feats], e_dw, TOL, 'dW rows')
    assert_close(db, dz.float().sum(0).bfloat16(), TOL, 'db')
    # Size-independent property at full size: the gradients are linear in dY.
    y3, dx3, dw3, db3, _ = run_layer(x, w, b, 'gelu', dy * 2)
    assert torch.equal(y3, y)
    torch.testing.assert_close(dw3.float(), 2 * dw.float(), rtol=2e-2, atol=1e-3)
    torch.testing.assert_close(db3.float(), 2 * db.float(), rtol=2e-2, atol=1e-3)
    torch.testing.assert_close(dx3.float(), 2 * dx.float(), rtol=2e-2, atol=1e-4)


@pytest.mark.parametrize('m', [1, 8, 32, 128])
def test_config4_skinny_fp16(m):
    """The skinny forward-only configuration at reduced N (fp16, forward only, K = 8192): the swap-AB stream-K kernel."""
    gen = torch.Generator().manual_seed(m)
    K, N = 8192, 4096
    x = torch.randn(m, K, generator=gen).half()
    w = (torch.randn(K, N, generator=gen) * 0.02).half()
    layer = make_layer(w, None, None, torch.float16)
    with torch.no_grad():
        y = layer(x.to(DEV))
    attorch_b200.check_status()
    assert _lib.load().ab200_last_path() == _lib.PATH_STREAMK
    e_y, _ = oracle.linear_forward(x, w, None, None)
    assert_close(y.cpu(), e_y, TOL, 'output')


@pytest.mark.parametrize('act_func', [None, 'silu'])
@pytest.mark.parametrize('m', [1, 8, 32, 100, 128])
def test_config4_full_width_fp16(m, act_func):
    """
    The skinny forward-only configuration at its full output width (N = 28672) and reduced K: from 8 rows on, the 112
    column blocks of 256 run as one wave of whole tiles with the fused epilogue; fewer rows keep the
    swap-AB stream-K kernel.  Both against the oracle.
    """
    gen = torch.Generator().manual_seed(100 + m)
    K, N = 512, 28672
    x = torch.randn(m, K, generator=gen).half()
    w = (torch.randn(K, N, generator=gen) * 0.05).half()
    b = torch.randn(N, generator=gen).half()
    layer = make_layer(w, b, act_func, torch.float16)
    with torch.no_grad():
        y = layer(x.to(DEV))
    attorch_b200.check_status()
    if torch.cuda.get_device_properties(0).multi_processor_count <= 186:
        expected = _lib.PATH_TCGEN05 if m >= 8 else _lib.PATH_STREAMK
        assert _lib.load().ab200_last_path() == expected
    e_y, _ = oracle.linear_forward(x, w, b, act_func)
    assert_close(y.cpu(), e_y, TOL, 'output')


def test_weight_gradient_in_row_blocks():
    """dW computed in four row blocks (as the data-parallel harness asks for) equals dW in one piece."""
    x, w, b, dy = seeded((512, 1024), 768, torch.bfloat16, seed=13)
    calls = []
    results = []
    for chunks in (1, 4):
        layer = make_layer(w, b, 'gelu', torch.bfloat16)
        layer.grad_ready = lambda i, n: calls.append((i, n))
        layer.dw_chunks = chunks
        xg = x.to(DEV).requires_grad_(True)
        layer(xg).backward(dy.to(DEV))
        attorch_b200.check_status()
        results.append((layer.weight.grad.cpu(), layer.bias.grad.cpu(), xg.grad.cpu()))
    assert calls == [(0, 1), (0, 4), (1, 4), (2, 4), (3, 4)]
    for a, c in zip(*results):
        assert torch.equal(a, c)


def test_shared_out_last_round_of_tiles(monkeypatch):
    """
    90 pair tiles on 74 CTA pairs with AB200_TAIL_MODE=2: the 16 tiles of the second round have their
    reductions shared out over all SMs (per-worker partial tiles summed in worker order by a
    finishing kernel).  Parity with the oracle, agreement of the forward output with the whole-tile
    schedule, and bit-repeatability.
    """
    monkeypatch.setenv('AB200_TAIL_MODE', '2')
    x, w, b, dy = seeded((2560, 1024), 2304, torch.bfloat16, seed=17)
    got = check_layer(x, w, b, 'gelu', dy)
    whole = run_layer(x, w, b, 'gelu', dy, flags=_lib.FLAG_WHOLE_TILES)
    torch.testing.assert_close(got[0].float(), whole[0].float(), rtol=1e-2, atol=1e-2)
    # The forward pass (hybrid schedule) and dX are bit-repeatable; dW [1024, 2304] over 2560 rows is
    # small enough to take the atomically summed stream-K path, whose addition order is not fixed.
    again = run_layer(x, w, b, 'gelu', dy)
    assert torch.equal(got[0], again[0]) and torch.equal(got[1], again[1])
    torch.testing.assert_close(got[2].float(), again[2].float(), rtol=1e-2, atol=1e-2)


def test_gemms_under_a_cta_limit():
    """With SMs held back for a collective the persistent GEMMs still cover every tile."""
    lib = _lib.load()
    x, w, b, dy = seeded((1536, 320), 768, torch.bfloat16, seed=19)
    previous = lib.ab200_set_gemm_cta_limit(100)
    try:
        check_layer(x, w, b, 'silu', dy)
    finally:
        assert lib.ab200_set_gemm_cta_limit(previous) == 100


def test_mlp_pair_shapes_of_config3():
    """The transformer MLP pair at reduced token count: 4096 -> 14336 (silu, no bias) -> 4096 (no bias)."""
    gen = torch.Generator().manual_seed(23)
    x = torch.randn(384, 4096, generator=gen).bfloat16()
    w_up = (torch.randn(4096, 14336, generator=gen) * 0.02).bfloat16()
    w_down = (torch.randn(14336, 4096, generator=gen) * 0.02).bfloat16()
    dy = (torch.randn(384, 4096, generator=gen) * 0.01).bfloat16()
    up = check_layer(x, w_up, None, 'silu', torch.randn(384, 14336, generator=gen).bfloat16())
    check_layer(up[0], w_down, None, None, dy)


def test_deferred_input_gradient():
    """
    The data-parallel harness may hold back the first layer's dX (the last product of backward) and
    launch it later: the input's gradient tensor is the buffer that product writes, and everything
    equals the undeferred run bit for bit.
    """
    from attorch_b200.dp import GradientBuckets
    x, w, b, dy = seeded((512, 256), 384, torch.bfloat16, seed=29)
    results = []
    for defer in (False, True):
        layer = make_layer(w, b, 'gelu', torch.bfloat16)
        buckets = GradientBuckets([layer], overlap=False, defer_first_input_grad=defer)
        xg = x.to(DEV).requires_grad_(True)
        layer(xg).backward(dy.to(DEV))
        if defer:
            assert len(buckets._deferred) == 1
            buckets.start_exchange()        # world size 1: nothing to exchange
            buckets.run_deferred()
            assert not buckets._deferred
        buckets.finish()
        attorch_b200.check_status()
        results.append((xg.grad.cpu(), layer.weight.grad.cpu(), layer.bias.grad.cpu()))
    for plain, deferred in zip(*results):
        assert torch.equal(plain, deferred)


@pytest.mark.gpu
def test_scratch_of_idle_streams_is_trimmed():
    """Per-stream scratch (status word, workspace) does not grow without bound: check_status() keeps the
    most recently used entries only, and a trimmed stream gets a fresh entry when it is used again."""
    import attorch_b200
    from attorch_b200 import linear_layer
    layer = attorch_b200.Linear(64, 64, act_func='relu')
    x = torch.randn(32, 64, device='cuda')
    streams = [torch.cuda.Stream() for _ in range(linear_layer._MAX_SCRATCH_ENTRIES + 8)]
    expected = layer(x)
    for stream in streams:
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            y = layer(x)
        torch.cuda.current_stream().wait_stream(stream)
        assert torch.equal(y, expected)
    assert len(linear_layer._scratch) > linear_layer._MAX_SCRATCH_ENTRIES
    attorch_b200.check_status()
    assert len(linear_layer._scratch) == linear_layer._MAX_SCRATCH_ENTRIES
    with torch.cuda.stream(streams[0]):                 # the oldest entry was dropped: a new one is made
        assert torch.equal(layer(x), expected)
    attorch_b200.check_status()
