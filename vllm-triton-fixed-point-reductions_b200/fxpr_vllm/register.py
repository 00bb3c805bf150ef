"""vLLM general-plugin entry point (``vllm.general_plugins`` ->
``fxpr_vllm.register:register``), idempotent, run once per worker process
(``fxpr_vllm/register.py:10-40`` of the reference)."""
from __future__ import annotations

import logging

from .config import get_runtime_config

logger = logging.getLogger("fxpr_vllm")

_done = False


def register() -> None:
    global _done
    if _done:
        return
    cfg = get_runtime_config()
    logger.info("fxpr_vllm (B200 kernels): int_bits=%d frac_bits=%d rms_norm=%s lm_head=%s",
                cfg.fxp_int_bits, cfg.fxp_frac_bits, cfg.enable_rms_norm, cfg.enable_lm_head)

    from vllm.model_executor.layers.quantization import register_quantization_config

    from . import monkey_patches
    from .quantisation_config import FixedPointConfig

    register_quantization_config("fixedpoint")(FixedPointConfig)
    monkey_patches.patch_attention_backend()
    steps = ["quant config 'fixedpoint'", "attention backend CUSTOM"]
    if cfg.enable_rms_norm:
        monkey_patches.patch_rms_norm()
        steps.append("RMSNorm")
    if cfg.enable_lm_head:
        steps.append("lm_head via gemm_fxp")
    if cfg.enable_sampler:
        monkey_patches.patch_sampler()
        steps.append("sampler log-softmax")
    logger.info("registered: %s", ", ".join(steps))
    _done = True
