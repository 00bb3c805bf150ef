"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (no dataset or checkpoint is involved anywhere: the
shapes stand in for Llama-3-8B geometry and weights are random)."""
from __future__ import annotations

import torch

LLAMA3_8B = dict(hidden=4096, ffn=14336, q_heads=32, kv_heads=8, head_dim=128, vocab=128256,
                 layers=32)


def _gen(seed: int, device) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed)


def rms_norm_inputs(rows=2048, hidden=4096, dtype=torch.float32, seed=0, device="cuda"):
    """x, residual ~ N(0,1); weight ~ N(1, 0.1)."""
    g = _gen(seed, device)
    x = torch.randn((rows, hidden), generator=g, device=device).to(dtype)
    r = torch.randn((rows, hidden), generator=g, device=device).to(dtype)
    w = (1.0 + 0.1 * torch.randn((hidden,), generator=g, device=device)).to(dtype)
    return x, r, w


def gemm_inputs(M=4096, N=4096, K=4096, dtype=torch.bfloat16, seed=1, device="cuda"):
    """A ~ N(0,1) [M,K]; B ~ N(0,0.02) stored (K,N) row-major like ``weight_native``."""
    g = _gen(seed, device)
    a = torch.randn((M, K), generator=g, device=device).to(dtype)
    b = (0.02 * torch.randn((K, N), generator=g, device=device)).to(dtype)
    return a, b


def paged_attention_inputs(seq_lens, q_lens, q_heads=32, kv_heads=8, head_dim=128, page=16,
                           dtype=torch.bfloat16, seed=2, device="cuda", extra_blocks=1):
    """Q/K/V ~ N(0,1); block table = random permutation of the physical pages."""
    g = _gen(seed, device)
    blocks = [-(-int(s) // page) for s in seq_lens]
    total = sum(blocks)
    kv = torch.randn((total + extra_blocks, 2, page, kv_heads, head_dim), generator=g,
                     device=device).to(dtype)
    perm = torch.randperm(total, generator=g, device=device).to(torch.int32) + extra_blocks
    bt = torch.zeros((len(seq_lens), max(blocks)), dtype=torch.int32, device=device)
    o = 0
    for r, nb in enumerate(blocks):
        bt[r, :nb] = perm[o:o + nb]
        o += nb
    qsl = torch.zeros(len(q_lens) + 1, dtype=torch.int32)
    qsl[1:] = torch.tensor(q_lens, dtype=torch.int32).cumsum(0)
    q = torch.randn((int(qsl[-1]), q_heads, head_dim), generator=g, device=device).to(dtype)
    sl = torch.tensor([int(s) for s in seq_lens], dtype=torch.int32, device=device)
    return q, kv, qsl.to(device), sl, bt


def decode_batch_lens(batch=64, lo=512, hi=8192, seed=3):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (batch,), generator=g).tolist()


def prefill_batch_lens(batch=16, lo=128, hi=4096, seed=4):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (batch,), generator=g).tolist()


def logits_inputs(rows=256, vocab=128256, dtype=torch.float32, seed=5, device="cuda"):
    """fp32 logits ~ N(0, variance 4)."""
    g = _gen(seed, device)
    return (2.0 * torch.randn((rows, vocab), generator=g, device=device)).to(dtype)
