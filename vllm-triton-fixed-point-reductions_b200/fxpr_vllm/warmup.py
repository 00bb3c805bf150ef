"""Warm-up hooks.

The reference uses these to JIT-compile and autotune its Triton kernels at load
time (``fxpr_vllm/warmup.py:19-182``).  The kernels here are compiled ahead of
time, so nothing needs compiling; the hooks keep their names and their
``FXPR_DISABLE_*_WARMUP`` switches and only do what must happen before CUDA-graph
capture: load the shared library, size the persistent split-K scratch and create
the per-device status word.  Like the reference's, they never raise.
"""
from __future__ import annotations

import logging

import torch

from .config import get_runtime_config

logger = logging.getLogger("fxpr_vllm")


def _capturing() -> bool:
    try:
        return torch.cuda.is_current_stream_capturing()
    except Exception:
        return False


def warmup_gemm(weight_native: torch.Tensor, fxp_int_bits: int, fxp_frac_bits: int) -> None:
    if get_runtime_config().disable_gemm_warmup or _capturing() or not weight_native.is_cuda:
        return
    try:
        from . import _lib, _native

        _native.load()
        # sized from the split-K policy's own bound (tens of MB), not from N: a
        # 128256-column lm_head must not pin gigabytes before the KV cache is sized
        need = _lib.gemm_scratch_policy_bytes(_lib._sm_count(weight_native.device), fxp_int_bits)
        _lib._get_gemm_scratch(weight_native.device, int(need))
        _lib._status_word(weight_native.device)
    except Exception as exc:  # warm-up must never break serving
        logger.warning("gemm warm-up skipped: %s", exc)


def warmup_rms_norm(hidden: int, dtype: torch.dtype, device: torch.device) -> None:
    if get_runtime_config().disable_rms_norm_warmup or _capturing():
        return
    try:
        from . import _native

        _native.load()
    except Exception as exc:
        logger.warning("rms_norm warm-up skipped: %s", exc)


def warmup_attention(num_heads, num_kv_heads, head_size, dtype, device, window_size=0,
                     logit_softcap=0.0, fxp_int_bits=32, fxp_frac_bits=16) -> None:
    if get_runtime_config().disable_attention_warmup or _capturing():
        return
    try:
        from . import _native

        _native.load()
    except Exception as exc:
        logger.warning("attention warm-up skipped: %s", exc)
