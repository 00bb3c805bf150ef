"""Runtime knobs read once from the environment.

Mirrors ``fxpr_vllm/config.py:26-73`` of the reference: the same variable
names, defaults (Q16.16 in int32) and warn-and-fall-back behaviour.  Two extra,
non-breaking knobs exist because the public ``gemm_fxp`` schema has no argument
for them: ``FXPR_GEMM_KTILE`` (K-tile = conversion granularity; 0 keeps the
reference's per-dtype default) and ``FXPR_GEMM_SPLIT_K`` (0 = automatic).
``FXPR_DISABLE_SAMPLER=1`` keeps vLLM's own ``log_softmax`` in the sampler (the
reference's README lists a sampler module but ships none, so this switch has no
counterpart there).
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass

DEFAULT_FXP_INT_BITS = 32
DEFAULT_FXP_FRAC_BITS = 16

logger = logging.getLogger("fxpr_vllm")


def _env_int(name: str, default: int) -> int:
    raw = os.getenv(name)
    if raw is None or raw == "":
        return default
    try:
        return int(raw)
    except ValueError:
        logger.warning("Ignoring malformed %s=%r; using default %d", name, raw, default)
        return default


def _env_flag(name: str) -> bool:
    return os.getenv(name) == "1"


@dataclass(frozen=True)
class FxpRuntimeConfig:
    fxp_int_bits: int = DEFAULT_FXP_INT_BITS
    fxp_frac_bits: int = DEFAULT_FXP_FRAC_BITS
    enable_rms_norm: bool = True
    enable_lm_head: bool = True
    enable_sampler: bool = True
    disable_attention_warmup: bool = False
    disable_gemm_warmup: bool = False
    disable_rms_norm_warmup: bool = False
    gemm_k_tile: int = 0
    gemm_split_k: int = 0


def _validated(name: str, allowed: tuple[int, ...], default: int) -> int:
    value = _env_int(name, default)
    if value not in allowed:
        logger.warning(
            "Invalid %s=%d; must be one of %s. Using default %d.",
            name, value, "/".join(str(a) for a in allowed), default,
        )
        return default
    return value


def load_runtime_config() -> FxpRuntimeConfig:
    return FxpRuntimeConfig(
        fxp_int_bits=_validated("FXPR_INT_BITS", (16, 32, 64), DEFAULT_FXP_INT_BITS),
        fxp_frac_bits=_validated("FXPR_FRAC_BITS", (8, 16, 32), DEFAULT_FXP_FRAC_BITS),
        enable_rms_norm=not _env_flag("FXPR_DISABLE_RMS_NORM"),
        enable_lm_head=not _env_flag("FXPR_DISABLE_LM_HEAD"),
        enable_sampler=not _env_flag("FXPR_DISABLE_SAMPLER"),
        disable_attention_warmup=_env_flag("FXPR_DISABLE_ATTENTION_WARMUP"),
        disable_gemm_warmup=_env_flag("FXPR_DISABLE_GEMM_WARMUP"),
        disable_rms_norm_warmup=_env_flag("FXPR_DISABLE_RMS_NORM_WARMUP"),
        gemm_k_tile=_validated("FXPR_GEMM_KTILE", (0, 64, 128), 0),
        gemm_split_k=_validated("FXPR_GEMM_SPLIT_K", (0, 1, 2, 4, 8, 16), 0),
    )


_runtime_config: FxpRuntimeConfig | None = None


def get_runtime_config() -> FxpRuntimeConfig:
    global _runtime_config
    if _runtime_config is None:
        _runtime_config = load_runtime_config()
    return _runtime_config


def reset_runtime_config() -> None:
    """Forget the cached config (tests that change the environment call this)."""
    global _runtime_config
    _runtime_config = None
