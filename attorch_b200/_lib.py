"""
ctypes binding of libattorch_b200.so (declared in include/attorch_b200.h).

There is no fallback: if the library is missing or does not load, every entry point raises.
"""

import ctypes
import os
from pathlib import Path
from typing import Optional

PKG_DIR = Path(__file__).resolve().parent
# The in-tree build, unless AB200_LIBRARY names another build of the same sources (A/B comparisons).
LIB_PATH = Path(os.environ['AB200_LIBRARY']) if os.environ.get('AB200_LIBRARY') else PKG_DIR / 'libattorch_b200.so'

# Element type ids (include/attorch_b200.h).
F32, F16, BF16 = 0, 1, 2

FLAG_FORCE_GENERIC = 1
FLAG_FORCE_TCGEN05 = 2
FLAG_FORCE_STREAMK = 4
FLAG_NO_STREAMK = 8
FLAG_NO_PAIR = 16
FLAG_NO_TMA_STORE = 32
FLAG_SAVE_DERIVATIVE = 64
FLAG_WHOLE_TILES = 128
FLAG_DROPOUT_PACKED = 256
FLAG_DERIVATIVE_FP16 = 512
FLAG_RESERVE_SMS_SHIFT = 16   # bits 16-23: SMs a GEMM call leaves free
ACT_SAVED_DERIVATIVE = 22
ACT_SAVED_DERIVATIVE_F16 = 23

PATH_TCGEN05, PATH_STREAMK, PATH_GENERIC = 1, 2, 3

_i64 = ctypes.c_int64
_int = ctypes.c_int
_ptr = ctypes.c_void_p
_f32 = ctypes.c_float

# name -> (restype, argtypes); one entry per symbol the header declares.
SIGNATURES = {
    'ab200_version': (_int, []),
    'ab200_error_string': (ctypes.c_char_p, [_int]),
    'ab200_last_path': (_int, []),
    'ab200_last_schedule': (_int, []),
    'ab200_launch_count': (_i64, []),
    'ab200_set_gemm_cta_limit': (_int, [_int]),
    'ab200_forward_workspace_bytes': (_i64, [_i64, _i64, _i64, _int]),
    'ab200_gemm_workspace_bytes': (_i64, [_i64, _i64, _i64]),
    'ab200_linear_forward': (_int, [_ptr, _ptr, _ptr, _ptr, _ptr,
                                    _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                    _int, _int, _int, _int, _f32,
                                    _ptr, _i64, _ptr, _ptr, _int]),
    'ab200_linear_forward_residual': (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                                             _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                             _int, _int, _int, _int, _f32,
                                             _ptr, _i64, _ptr, _ptr, _int]),
    'ab200_gated_linear_forward': (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                          _i64, _int, _int, _int, _int, _f32, _ptr, _ptr, _int]),
    'ab200_act_backward_workspace_bytes': (_i64, [_i64, _i64]),
    'ab200_act_backward': (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64,
                                  _int, _int, _int, _f32, _ptr, _i64, _ptr]),
    'ab200_act_backward_static': (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64,
                                         _int, _int, _int, _f32, _ptr]),
    'ab200_act_backward_static_max_floats': (_i64, []),
    'ab200_linear_backward_input': (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64,
                                           _i64, _i64, _i64, _i64, _i64,
                                           _int, _int, _ptr, _i64, _ptr, _ptr, _int]),
    'ab200_linear_backward_weight': (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64,
                                            _i64, _i64, _i64, _i64, _i64,
                                            _int, _int, _ptr, _i64, _ptr, _ptr, _int]),
    'ab200_act_forward': (_int, [_ptr, _ptr, _i64, _int, _int, _f32, _f32, ctypes.c_uint32, _ptr, _int]),
    'ab200_act_input_grad': (_int, [_ptr, _ptr, _ptr, _i64, _int, _int, _f32, _f32, ctypes.c_uint32, _ptr,
                                    _int]),
    'ab200_glu_forward': (_int, [_ptr, _ptr, _i64, _i64, _int, _int, _f32, _ptr]),
    'ab200_glu_backward': (_int, [_ptr, _ptr, _ptr, _i64, _i64, _int, _int, _f32, _ptr]),
    'ab200_dropout_uniform': (_f32, [ctypes.c_uint32, ctypes.c_uint64, _int]),
    'ab200_dropout_threshold': (ctypes.c_uint32, [_f32, _int]),
    'ab200_cast_2d': (_int, [_ptr, _ptr, _i64, _i64, _i64, _i64, _int, _int, _ptr]),
    'ab200_cross_entropy_workspace_bytes': (_i64, [_i64]),
    'ab200_cross_entropy_forward': (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _int, _int, _int,
                                           _ptr, _i64, _ptr]),
    'ab200_cross_entropy_backward': (_int, [_ptr, _int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64,
                                            _i64, _int, _int, _int, _ptr]),
    'ab200_linear_backward_input_fused': (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                                 _int, _int, _ptr, _ptr]),
    'ab200_layer_norm_forward': (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _int, _int, _int,
                                        _f32, _ptr]),
    'ab200_layer_norm_workspace_bytes': (_i64, [_i64, _i64]),
    'ab200_layer_norm_backward': (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64,
                                         _int, _int, _int, _int, _ptr, _i64, _ptr, _ptr]),
    'ab200_multimem_all_reduce': (_int, [_ptr, _i64, _int, _int, _int, _ptr, _int, _ptr, _ptr]),
    'ab200_collective_flag_bytes': (_i64, []),
}

_lib: Optional[ctypes.CDLL] = None


class LibraryError(RuntimeError):
    """Raised when libattorch_b200.so is missing, fails to load, or a call is rejected."""


def load() -> ctypes.CDLL:
    """Loads the library once and attaches the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise LibraryError(
            f'{LIB_PATH} not found: build it with `python -m attorch_b200.build` '
            '(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.')
    try:
        lib = ctypes.CDLL(str(LIB_PATH))
    except OSError as error:
        raise LibraryError(f'cannot load {LIB_PATH}: {error}') from error
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            func = getattr(lib, name)
        except AttributeError as error:
            raise LibraryError(f'{LIB_PATH} does not export {name}') from error
        func.restype = restype
        func.argtypes = argtypes
    _lib = lib
    return lib


def error_string(code: int) -> str:
    return load().ab200_error_string(code).decode()


def check(code: int, what: str) -> None:
    """Raises LibraryError for a negative return code of an entry point."""
    if code != 0:
        raise LibraryError(f'{what} failed: {error_string(code)} (code {code})')
