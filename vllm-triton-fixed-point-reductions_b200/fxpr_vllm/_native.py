"""ctypes binding of ``libfxpr_b200.so`` (the C ABI in ``include/fxpr_b200.h``).

There is no fallback: if the library is missing the first kernel call raises.
The library is built in-tree by ``build.py`` next to this package.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_PKG_ROOT = Path(__file__).resolve().parent.parent


def _find_lib() -> Path:
    """``FXPR_B200_LIB`` if set, else a copy packaged beside this module (wheel
    installs), else the in-tree build output ``../lib/``."""
    env = os.environ.get("FXPR_B200_LIB")
    if env:
        return Path(env)
    beside = Path(__file__).resolve().parent / "libfxpr_b200.so"
    return beside if beside.exists() else _PKG_ROOT / "lib" / "libfxpr_b200.so"


LIB_PATH = _find_lib()

FXPR_OK = 0
FXPR_ERR_BAD_ARG = -1
FXPR_ERR_UNSUPPORTED = -2
FXPR_ERR_SCRATCH = -3
FXPR_ERR_CUDA = -4
FXPR_ERR_TIMEOUT = -5
FXPR_ERR_ARCH = -6

FXPR_F16, FXPR_BF16, FXPR_F32, FXPR_F64 = 0, 1, 2, 3
DTYPE_CODE = {
    torch.float16: FXPR_F16,
    torch.bfloat16: FXPR_BF16,
    torch.float32: FXPR_F32,
    torch.float64: FXPR_F64,
}

GEMM_FORCE_PORTABLE = 1
GEMM_FORCE_EXACT_TC = 2
GEMM_NO_SKINNY = 8
GEMM_NO_CLUSTER = 16
GEMM_PAIR = 512
GEMM_SILU_MUL = 1024
GEMM_WEIGHTS_STATIC = 2048
TP_LOCAL_RESIDUAL = 1
GEMM_TILE_N256 = 64
GEMM_TILE_N128 = 128
ATTN_CAUSAL = 1
ATTN_FORCE_PORTABLE = 2
ATTN_EXACT_CONVERT = 4
ATTN_NO_TCGEN05 = 8

_c = ctypes
_vp, _i, _i64, _f, _d = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_float, _c.c_double

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "fxpr_version": (_i, []),
    "fxpr_status_string": (_c.c_char_p, [_i]),
    "fxpr_last_error": (_c.c_char_p, []),
    "fxpr_float_to_fixed": (_i, [_vp, _i, _vp, _i, _i, _i64, _vp]),
    "fxpr_fixed_to_float": (_i, [_vp, _i, _vp, _i, _i, _i64, _vp]),
    "fxpr_rms_norm": (_i, [_vp, _vp, _vp, _vp, _i, _i64, _i64, _f, _i, _vp]),
    "fxpr_rms_norm_from_int": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _i64, _i64, _f, _i, _i, _vp]),
    "fxpr_log_softmax": (_i, [_vp, _i, _vp, _i64, _i64, _i, _vp]),
    "fxpr_tp_buffer_bytes": (_i, [_i64, _i64, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "fxpr_tp_alloc": (_i, [_i64, _vp, _vp]),
    "fxpr_tp_open": (_i, [_vp, _vp]),
    "fxpr_tp_close": (_i, [_vp]),
    "fxpr_tp_free": (_i, [_vp]),
    "fxpr_tp_reduce_norm": (_i, [_vp, _i, _i, _vp, _i64, _i64, _i64, _i64, _i, _vp, _vp, _i, _i64, _i64, _f,
                                 _i, _i, _i64, _i, _vp, _vp]),
    "fxpr_rope_kv_write": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i, _i, _i, _i,
                                _i64, _i64, _i64, _i64, _vp]),
    "fxpr_silu_mul": (_i, [_vp, _i, _vp, _i64, _i64, _vp]),
    "fxpr_silu_mul_pairs": (_i, [_vp, _i, _vp, _i64, _i64, _vp]),
    "fxpr_gemm_scratch_bytes": (_i64, [_i64, _i64, _i, _i]),
    "fxpr_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64,
                       _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _i,
                       _vp, _i64, _vp, _vp, _vp]),
    "fxpr_gemm_argmax": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                              _i, _i, _i, _i, _vp, _vp]),
    "fxpr_gemm_epilogue_from_int": (_i, [_vp, _i, _vp, _vp, _i, _i64, _i64, _i64, _i, _vp]),
    "fxpr_attention_scratch_bytes": (_i64, [_i64, _i, _i, _i, _i]),
    "fxpr_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                            _i, _i64, _i, _i, _i, _i, _i,
                            _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                            _i, _i, _d, _d, _i, _i, _i, _i, _vp, _i64, _vp, _vp]),
    "fxpr_attention_static_scratch_capacity": (_i64, []),
    "fxpr_attention_static_scratch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                           _i, _i64, _i, _i, _i, _i, _i,
                                           _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                           _i, _i, _d, _d, _i, _i, _i, _i, _vp, _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"fxpr_vllm: CUDA library {LIB_PATH} is missing; run "
                f"`python {_PKG_ROOT / 'build.py'}` (there is no CPU or Triton fallback)"
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    """Map a C status to the exception types the reference raises for the same
    class of error (ValueError / TypeError / RuntimeError)."""
    if status == FXPR_OK:
        return
    lib = load()
    msg = lib.fxpr_status_string(status).decode()
    detail = lib.fxpr_last_error().decode()
    text = f"{what}: {msg}" + (f" [{detail}]" if detail and status == FXPR_ERR_CUDA else "")
    if status == FXPR_ERR_BAD_ARG:
        raise ValueError(text)
    if status == FXPR_ERR_UNSUPPORTED:
        raise TypeError(text)
    raise RuntimeError(text)


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()
