"""ctypes binding of librmsnorm_linear.so (the C ABI in include/rmsnorm_linear.h).

There is no fallback: if the library is missing or fails to load, importing
the operator raises.
"""
from __future__ import annotations

import ctypes
import os

from ._build import LIB_PATH

RL_OK = 0
RL_ERR_NULL_POINTER = -1
RL_ERR_BAD_SHAPE = -2
RL_ERR_ALIGNMENT = -3
RL_ERR_BAD_DTYPE = -4
RL_ERR_WORKSPACE = -5
RL_ERR_UNSUPPORTED_ARCH = -6
RL_ERR_BAD_VARIANT = -7
RL_ERR_TENSOR_MAP = -8
RL_ERR_DEVICE_TIMEOUT = -9
RL_ERR_STATIC_SCRATCH = -10
RL_ERR_CUDA = -1000

RL_W_BF16 = 0
RL_W_E4M3 = 1

VARIANTS = {
    "auto": 0,
    "prefill_ts_n192": 1,
    "prefill_ss_n192": 2,
    "prefill_ss_n256": 3,
    "prefill_ts_n128": 4,
    "prefill_ss_n128": 5,
    "prefill_pair_n256": 9,
    "prefill_pair_n192": 10,
    "prefill_pair_direct": 11,
    "prefill_pair_prestats": 14,
    "prefill_pair_prestats_whole": 15,
    "prefill_pair_direct_prestats": 16,
    "prefill_pair_prescaled": 17,
    "prefill_pair_wide": 18,
    "decode": 20,
    "auto_whole": 30,
}
VARIANT_NAMES = {v: k for k, v in VARIANTS.items()}

# every symbol include/rmsnorm_linear.h declares: (name, restype, argtypes)
_vp, _i, _i64, _sz, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t, ctypes.c_float
SYMBOLS = [
    ("rl_version", _i, []),
    ("rl_error_string", ctypes.c_char_p, [_i]),
    ("rl_workspace_bytes", _sz, [_i, _i, _i, _i]),
    ("rl_plan_tail_split", _i, [_i, _i, _i, _i, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]),
    ("rl_select_variant", _i, [_i, _i, _i, _i, _i]),
    ("rl_workspace_init", _i, [_vp, _sz, _vp]),
    ("rl_rmsnorm_linear_bf16", _i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, _f, _vp, _sz, _i, _vp]),
    ("rl_rmsnorm_linear_fp8w", _i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, _f, _vp, _sz, _i, _vp]),
    ("rl_row_stats", _i, [_vp, _vp, _vp, _vp, _i, _i, _i64, _f, _vp]),
    ("rl_quantize_rows_e4m3", _i, [_vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _f, _vp]),
    ("rl_rmsnorm_linear_bf16_noalloc", _i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, _f, _vp]),
    ("rl_rmsnorm_swiglu_bf16", _i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, _f, _vp, _sz, _vp]),
    ("rl_gemm_bf16", _i, [_vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, _vp, _sz, _vp]),
    ("rl_lora_linear_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _vp, _sz, _vp]),
    ("rl_selftest_wait_timeout", _i, [_vp, _sz, ctypes.c_ulonglong, _vp]),
    ("rl_read_status", _i, [_vp, ctypes.POINTER(ctypes.c_int)]),
]

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it is not there."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m kernel_benchmarking_b200._build` "
                "(there is no CPU or PyTorch fallback for this operator)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, restype, argtypes in SYMBOLS:
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def error_string(code: int) -> str:
    return load().rl_error_string(code).decode()


def check(code: int, what: str) -> None:
    """Translate an RL_ERR_* code into the Python exception the reference's callers expect:
    argument problems -> ValueError, everything else -> RuntimeError."""
    if code == RL_OK:
        return
    msg = f"{what}: {error_string(code)} (code {code})"
    if code in (RL_ERR_NULL_POINTER, RL_ERR_BAD_SHAPE, RL_ERR_ALIGNMENT, RL_ERR_BAD_DTYPE, RL_ERR_BAD_VARIANT,
                RL_ERR_STATIC_SCRATCH):
        raise ValueError(msg)
    raise RuntimeError(msg)
