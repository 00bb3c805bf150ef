"""Hooks into vLLM: swap the RMSNorm class and register the attention backend
under ``CUSTOM`` (what ``fxpr_vllm/monkey_patches.py:9-43`` of the reference does),
and route the sampler's log-softmax through ``log_softmax_fxp``."""
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


def patch_sampler() -> None:
    """``Sampler.compute_logprobs`` (vllm/v1/sample/sampler.py: ``logits.log_softmax(dim=-1,
    dtype=float32)``, whose float sum over the vocabulary depends on the reduction order)
    becomes the fixed-point log-softmax: exact row maximum, ``sum_i Q(exp(x_i - max))`` as
    an integer sum, one ``log``.  CUDA logits only; anything else keeps vLLM's own code."""
    import torch
    from vllm.v1.sample.sampler import Sampler

    from . import library_ops as ops
    from .config import get_runtime_config

    if getattr(Sampler.compute_logprobs, "_fxpr_patched", False):
        return
    original = Sampler.compute_logprobs
    frac_bits = get_runtime_config().fxp_frac_bits
    io_dtypes = (torch.float16, torch.bfloat16, torch.float32)

    def compute_logprobs(logits: torch.Tensor) -> torch.Tensor:
        if logits.is_cuda and logits.dtype in io_dtypes:
            return ops.log_softmax_fxp(logits, frac_bits)
        return original(logits)

    compute_logprobs._fxpr_patched = True
    compute_logprobs._fxpr_original = original
    Sampler.compute_logprobs = staticmethod(compute_logprobs)
