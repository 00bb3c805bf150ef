"""Thin wrappers the GPU tests share (the counterpart of the reference's
``fxpr_vllm/_tests/fixed_point_helpers.py``)."""
from __future__ import annotations

import torch

import fxpr_vllm  # noqa: F401  (registers torch.ops.fxpr)

INT_BITS = {torch.int16: 16, torch.int32: 32, torch.int64: 64}
FLOAT_BITS = {torch.float16: 16, torch.float32: 32, torch.float64: 64}
RCP_LN2 = 1.4426950408889634


def float_to_fixed(x, out, frac_bits=16):
    return torch.ops.fxpr.float_to_fixed(x.contiguous(), INT_BITS[out], int(frac_bits))


def fixed_to_float(x, out, frac_bits=16):
    return torch.ops.fxpr.fixed_to_float(x.contiguous(), FLOAT_BITS[out], int(frac_bits))


def gemm(a, b, bias=None, int_bits=32, frac_bits=16):
    return torch.ops.fxpr.gemm_fxp(a, b, bias, int(int_bits), int(frac_bits))


def make_paged_kv(seq_lens, num_kv_heads, head_dim, page, dtype, gen, device="cuda", shuffle=True):
    """Random paged KV cache + shuffled block table for the given sequence lengths."""
    blocks = [-(-int(s) // page) for s in seq_lens]
    total = sum(blocks)
    kv = torch.randn((total + 1, 2, page, num_kv_heads, head_dim), generator=gen,
                     dtype=torch.float32).to(dtype)
    order = (torch.randperm(total, generator=gen) if shuffle else torch.arange(total)) + 1
    bt = torch.zeros((len(seq_lens), max(blocks)), dtype=torch.int32)
    o = 0
    for r, nb in enumerate(blocks):
        bt[r, :nb] = order[o:o + nb].to(torch.int32)
        o += nb
    return kv.to(device), bt.to(device)


def run_attention(q, kv, qsl, seq_lens, bt, max_q, *, causal=True, scale=None, int_bits=32,
                  frac_bits=16, splits=1, alibi=None, softcap=0.0, window=0):
    o = torch.empty_like(q)
    torch.ops.fxpr.unified_attention_fxp(q, kv, o, qsl, seq_lens, bt, int(max_q), alibi, causal,
                                         scale, int_bits, frac_bits, float(softcap), int(window),
                                         int(splits))
    return o
