"""
Host-side tests that need no GPU: the C-ABI library loads and exports every symbol the header
declares, argument validation of the entry points (host checks run before any launch), the
activation-string parser, the dtype rule and the no-fallback guarantee.
"""

import ctypes
import re
from pathlib import Path

import pytest
import torch

import attorch_b200
from attorch_b200 import _lib, acts
from attorch_b200 import build as builder

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / 'include' / 'attorch_b200.h'


@pytest.fixture(scope='module')
def lib():
    builder.build()
    return _lib.load()


def declared_functions():
    text = re.sub(r'/\*.*?\*/', '', HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r'\b(ab200_\w+)\s*\(', text)))


def test_header_symbols_exported(lib):
    names = declared_functions()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f'{name} is declared in the header but not exported'
    assert sorted(_lib.SIGNATURES) == names, 'ctypes prototypes and header disagree'


def test_header_constants_match_python():
    text = HEADER.read_text()
    defines = dict(re.findall(r'#define\s+(AB200_\w+)\s+\(?(-?\d+)\)?', text))
    for name, ident in acts.ACT_IDS.items():
        macro = 'AB200_ACT_' + ('NONE' if name is None else name.upper())
        assert int(defines[macro]) == ident
    assert int(defines['AB200_F32']) == _lib.F32
    assert int(defines['AB200_F16']) == _lib.F16
    assert int(defines['AB200_BF16']) == _lib.BF16
    assert int(defines['AB200_FLAG_FORCE_GENERIC']) == _lib.FLAG_FORCE_GENERIC
    assert int(defines['AB200_FLAG_FORCE_TCGEN05']) == _lib.FLAG_FORCE_TCGEN05
    assert int(defines['AB200_FLAG_FORCE_STREAMK']) == _lib.FLAG_FORCE_STREAMK
    assert int(defines['AB200_FLAG_NO_STREAMK']) == _lib.FLAG_NO_STREAMK
    assert int(defines['AB200_FLAG_NO_PAIR']) == _lib.FLAG_NO_PAIR
    assert int(defines['AB200_FLAG_NO_TMA_STORE']) == _lib.FLAG_NO_TMA_STORE
    assert int(defines['AB200_FLAG_SAVE_DERIVATIVE']) == _lib.FLAG_SAVE_DERIVATIVE
    assert int(defines['AB200_FLAG_WHOLE_TILES']) == _lib.FLAG_WHOLE_TILES
    assert int(defines['AB200_FLAG_DROPOUT_PACKED']) == _lib.FLAG_DROPOUT_PACKED
    assert int(defines['AB200_FLAG_DERIVATIVE_FP16']) == _lib.FLAG_DERIVATIVE_FP16
    assert int(defines['AB200_ACT_SAVED_DERIVATIVE_F16']) == _lib.ACT_SAVED_DERIVATIVE_F16
    assert int(defines['AB200_ACT_SAVED_DERIVATIVE']) == _lib.ACT_SAVED_DERIVATIVE


def test_version_and_error_strings(lib):
    assert lib.ab200_version() == 1000
    assert _lib.error_string(0) == 'ok'
    for code in range(-12, 5):
        assert _lib.error_string(code) != 'unknown code'
    assert _lib.error_string(99) == 'unknown code'


def test_argument_validation_without_gpu(lib):
    """Host checks reject bad arguments before anything is launched (no device needed)."""
    fake = ctypes.c_void_p(0x1000)
    def fwd(M=4, K=8, N=8, op=2, out=2, act=0, x=fake, o=fake, ld_out=8):
        return lib.ab200_linear_forward(x, fake, None, None, o, M, K, N, K, 1, N, 1, N, ld_out,
                                        op, out, 0, act, 0.0, None, 0, None, None, 0)
    assert fwd(M=-1) == -2
    assert fwd(op=7) == -3
    assert fwd(act=22) == -4
    assert fwd(x=None) == -1
    assert fwd(o=None) == -1
    assert fwd(ld_out=4) == -5
    assert fwd(M=2 ** 31) == -9
    assert fwd(M=0) == 0            # empty batch: nothing to launch
    # The residual variant: same checks, plus the residual's row pitch.
    def fwd_res(ld_res, residual=fake, M=4):
        return lib.ab200_linear_forward_residual(fake, fake, None, None, fake, residual, M, 8, 8, 8, 1, 8, 1, 8, 8,
                                                 ld_res, 2, 2, 0, 0, 0.0, None, 0, None, None, 0)
    assert fwd_res(4) == -5
    assert fwd_res(4, residual=None, M=0) == 0
    assert fwd_res(8, M=-1) == -2
    assert lib.ab200_act_backward(fake, None, fake, None, 4, 8, 8, 8, 8, 2, 2, 5, 0.0, None, 0, None) == -1
    assert lib.ab200_act_backward(fake, fake, fake, fake, 4, 8, 8, 8, 8, 2, 2, 5, 0.0, None, 0, None) == -6
    assert lib.ab200_cast_2d(fake, fake, -1, 2, 2, 1, 0, 2, None) == -2
    assert lib.ab200_linear_backward_input(fake, fake, None, 4, 8, 8, 8, 1, 8, 1, 8, 2, 2, None, 0, None, None, 0) == -1
    assert lib.ab200_linear_backward_weight(fake, fake, fake, 4, 8, 8, 8, 1, 8, 1, 4, 2, 2, None, 0, None, None, 0) == -5


def test_collective_argument_validation_without_gpu(lib):
    """The all-reduce entry point rejects bad arguments on the host; a world of one is a no-op."""
    fake = ctypes.c_void_p(0x1000)
    def reduce(ptr=fake, numel=64, dtype=2, rank=0, world=2, flags=fake, status=fake):
        return lib.ab200_multimem_all_reduce(ptr, numel, dtype, rank, world, flags, 8, status, None)
    assert reduce(world=1) == 0 and reduce(numel=0) == 0
    assert reduce(numel=-1) == -2 and reduce(rank=2) == -2 and reduce(world=0) == -2
    assert reduce(world=17, rank=3) == -9
    assert reduce(dtype=5) == -3
    assert reduce(ptr=None) == -1 and reduce(flags=None) == -1 and reduce(status=None) == -1
    assert reduce(numel=63) == -5                            # 126 bytes: not whole 16-byte units
    assert reduce(ptr=ctypes.c_void_p(0x1008)) == -5         # misaligned base
    assert lib.ab200_collective_flag_bytes() == (32 * 16 + 32) * 4
    # The reservation field of the GEMM flags: bits 16-23.
    assert _lib.FLAG_RESERVE_SMS_SHIFT == 16


def test_workspace_sizes(lib):
    assert lib.ab200_forward_workspace_bytes(4, 8192, 28672, 0) == 4 * 28672 * 4
    # From 8 rows on a wide output runs as one wave of whole tiles: no scratch.
    assert lib.ab200_forward_workspace_bytes(8, 8192, 28672, 0) == 0
    assert lib.ab200_forward_workspace_bytes(8, 8192, 4096, 0) == 8 * 4096 * 4
    assert lib.ab200_forward_workspace_bytes(8192, 4096, 4096, 0) == 2 * 148 * 128 * 256 * 4
    assert lib.ab200_forward_workspace_bytes(300, 264, 520, _lib.FLAG_FORCE_STREAMK) == 300 * 520 * 4
    assert lib.ab200_forward_workspace_bytes(8, 64, 64, _lib.FLAG_NO_STREAMK) == 0
    # A 16 x 96 weight gradient over 131072 rows is one tile: its reduction is shared out.
    assert lib.ab200_gemm_workspace_bytes(16, 96, 131072) == 16 * 96 * 4
    assert lib.ab200_gemm_workspace_bytes(4096, 4096, 8192) == 2 * 148 * 128 * 256 * 4
    assert lib.ab200_gemm_workspace_bytes(256, 256, 8192) == 0
    assert lib.ab200_act_backward_workspace_bytes(8192, 4096) == 64 * 4096 * 4
    assert lib.ab200_act_backward_workspace_bytes(1, 16) == 64


@pytest.mark.parametrize('text,expected', [
    (None, (None, None)), ('relu', ('relu', None)), ('relu6', ('relu6', None)),
    ('leaky_relu_0.01', ('leaky_relu', 0.01)), ('elu_1', ('elu', 1.0)),
    ('hardshrink_0.5', ('hardshrink', 0.5)), ('geluapprox', ('geluapprox', None)),
])
def test_parse_act_func(text, expected):
    assert acts.parse_act_func(text) == expected


@pytest.mark.parametrize('text', ['leaky_relu', 'swish', 'elu', 'relu_2', 'soft_plus'])
def test_parse_act_func_rejects(text):
    with pytest.raises(ValueError):
        acts.parse_act_func(text)


def test_act_table_matches_oracle():
    from oracle import linear_oracle as oracle
    names = {oracle.parse_act_func(a)[0] for a in oracle.ALL_ACT_FUNCS}
    assert names == set(acts.ACT_IDS)
    assert sorted(acts.ACT_IDS.values()) == list(range(22))


def test_output_dtype_rule():
    assert attorch_b200.get_output_dtype(torch.float32) is torch.float32
    assert attorch_b200.get_output_dtype(torch.bfloat16) is torch.bfloat16
    if torch.cuda.is_available():     # CUDA autocast switches itself off on a machine without CUDA
        with torch.autocast('cuda', dtype=torch.float16):
            assert attorch_b200.get_output_dtype(torch.float32) is torch.float16
        with torch.autocast('cuda', dtype=torch.bfloat16):
            assert attorch_b200.get_output_dtype(torch.float32) is torch.bfloat16


def test_module_surface_and_no_cpu_fallback():
    layer = attorch_b200.Linear(12, 20, act_func='gelu', device='cpu')
    assert isinstance(layer, torch.nn.Linear)
    assert layer.weight.shape == (12, 20) and layer.bias.shape == (20,)
    assert set(layer.state_dict()) == {'weight', 'bias'}
    assert 'in_features=12' in repr(layer)
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        layer(torch.randn(3, 12))
    with pytest.raises(AssertionError, match='Incompatible input'):
        layer(torch.randn(3, 11))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, '_lib', None)
    monkeypatch.setattr(_lib, 'LIB_PATH', tmp_path / 'libattorch_b200.so')
    with pytest.raises(_lib.LibraryError, match='no CPU or PyTorch fallback'):
        _lib.load()
