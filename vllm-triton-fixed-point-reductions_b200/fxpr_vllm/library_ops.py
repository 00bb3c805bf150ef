"""Shape/dtype-only ("fake") implementations so Dynamo / torch.compile can trace
through the opaque ``fxpr`` ops, plus module-level aliases.

Same contract as ``fxpr_vllm/library_ops.py:28-78`` of the reference: casts map
the dtype and keep the shape, the norms return ``empty_like(x)``, the GEMM
returns ``a.new_empty((M, N))`` and attention returns nothing (it writes ``o``).
"""
from __future__ import annotations

import torch

from . import _lib  # noqa: F401  (defines the schemas)

_INT_BY_BITS = {16: torch.int16, 32: torch.int32, 64: torch.int64}
_FLOAT_BY_BITS = {16: torch.float16, 32: torch.float32, 64: torch.float64}


def _lookup(table: dict, bits: int, what: str) -> torch.dtype:
    try:
        return table[int(bits)]
    except KeyError:
        raise ValueError(f"{what} must be 16/32/64, got {bits}") from None


def _fake(name: str):
    return torch.library.register_fake(f"fxpr::{name}")


@_fake("float_to_fixed")
def _(x, int_bits, fxp_frac_bits):
    return torch.empty_like(x, dtype=_lookup(_INT_BY_BITS, int_bits, "int_bits"))


@_fake("fixed_to_float")
def _(x, float_bits, fxp_frac_bits):
    return torch.empty_like(x, dtype=_lookup(_FLOAT_BY_BITS, float_bits, "float_bits"))


@_fake("rms_norm_fxp")
def _(x, weight_fp32, eps):
    return torch.empty_like(x)


@_fake("rms_norm_fxp_residual")
def _(x, residual, weight_fp32, eps):
    return torch.empty_like(x)


@_fake("rms_norm_fxp_from_int")
def _(acc, residual, weight, bias, eps, gemm_frac_bits):
    return torch.empty_like(residual)


@_fake("gemm_fxp")
def _(a, b, bias, fxp_int_bits, fxp_frac_bits):
    return a.new_empty((a.shape[0], b.shape[1]))


@_fake("unified_attention_fxp")
def _(q, kv_cache, o, query_start_loc, seq_lens, block_table, max_query_len, alibi_slopes,
      is_causal, softmax_scale, fxp_int_bits, fxp_frac_bits, logit_softcap, window_size,
      num_kv_splits):
    return None


@_fake("log_softmax_fxp")
def _(x, fxp_frac_bits):
    return torch.empty_like(x, dtype=torch.float32)


@_fake("gemm_fxp_int")
def _(a, b, fxp_int_bits, fxp_frac_bits):
    return a.new_empty((a.shape[0], b.shape[1]),
                       dtype=_lookup(_INT_BY_BITS, fxp_int_bits, "fxp_int_bits"))


@_fake("gemm_fxp_epilogue")
def _(c_int, bias, out_dtype, fxp_frac_bits):
    return c_int.new_empty(c_int.shape, dtype=out_dtype)


gemm_fxp = torch.ops.fxpr.gemm_fxp
rms_norm_fxp = torch.ops.fxpr.rms_norm_fxp
rms_norm_fxp_residual = torch.ops.fxpr.rms_norm_fxp_residual
rms_norm_fxp_from_int = torch.ops.fxpr.rms_norm_fxp_from_int
float_to_fixed = torch.ops.fxpr.float_to_fixed
fixed_to_float = torch.ops.fxpr.fixed_to_float
unified_attention_fxp = torch.ops.fxpr.unified_attention_fxp
log_softmax_fxp = torch.ops.fxpr.log_softmax_fxp
gemm_fxp_int = torch.ops.fxpr.gemm_fxp_int
gemm_fxp_epilogue = torch.ops.fxpr.gemm_fxp_epilogue
