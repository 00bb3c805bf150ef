"""``DeterministicRMSNorm``: vLLM's RMSNorm module routed through the fixed-point
kernel (class and behaviour of ``fxpr_vllm/rms_norm.py:9-27`` in the reference).

Both of vLLM's dispatch targets are bound (``forward_native`` is what runs under
torch.compile, ``forward_cuda`` otherwise); leaving either unbound would silently
fall back to vLLM's batch-variant implementation.  With a residual the op adds in
place and the module returns ``(normed, residual)``.
"""
from __future__ import annotations

import torch
from vllm.model_executor.layers.layernorm import RMSNorm

from . import library_ops as ops


class DeterministicRMSNorm(RMSNorm):
    def _forward_fxp(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        eps = self.variance_epsilon
        if residual is None:
            return ops.rms_norm_fxp(x, self.weight, eps)
        normed = ops.rms_norm_fxp_residual(x, residual, self.weight, eps)
        return normed, residual

    forward_cuda = _forward_fxp
    forward_native = _forward_fxp
