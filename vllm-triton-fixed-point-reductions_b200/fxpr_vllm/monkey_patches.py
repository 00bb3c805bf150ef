"""Hooks into vLLM: swap the RMSNorm class and register the attention backend
under ``CUSTOM`` (what ``fxpr_vllm/monkey_patches.py:9-43`` of the reference does)."""
from __future__ import annotations

import logging
import sys

logger = logging.getLogger("fxpr_vllm")

_MODEL_MODULE_PREFIX = "vllm.model_executor.models."


def patch_rms_norm() -> None:
    import vllm.model_executor.layers.layernorm as layernorm_mod
    from vllm.model_executor.custom_op import op_registry, op_registry_oot

    from .rms_norm import DeterministicRMSNorm

    DeterministicRMSNorm.name = "rms_norm"
    for registry, key in ((op_registry, "rms_norm"), (op_registry_oot, "RMSNorm")):
        registry[key] = DeterministicRMSNorm
    layernorm_mod.RMSNorm = DeterministicRMSNorm

    # A model module imported before this point did `from ...layernorm import RMSNorm`
    # and holds the original class; it cannot be fixed from here, only reported.
    already = sum(1 for name in sys.modules if name.startswith(_MODEL_MODULE_PREFIX))
    if already:
        logger.warning(
            "patched RMSNorm but %d model module(s) already imported; those still use the original",
            already,
        )


def patch_attention_backend() -> None:
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    from .attention_backend import DeterministicAttentionBackend as backend

    register_backend(AttentionBackendEnum.CUSTOM,
                     class_path=f"{backend.__module__}.{backend.__qualname__}")
