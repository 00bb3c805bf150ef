"""Seeded inputs of the reference-fixture cases.  Used by the script that runs the
reference plugin's own Triton kernels on a B200 (``make_reference_fixtures.py``) and by
the GPU test that compares this repository's kernels with what the reference produced.
Inputs are generated on the CPU with ``torch.Generator`` so both sides see the same bits."""
from __future__ import annotations

import torch


def _g(seed):
    return torch.Generator().manual_seed(seed)


def cast_cases():
    out = []
    for i, (dt, bits, frac) in enumerate([(torch.float32, 32, 16), (torch.float16, 16, 8),
                                          (torch.float32, 64, 32), (torch.float64, 32, 8),
                                          (torch.float32, 64, 16)]):
        x = (torch.randn(5000, generator=_g(100 + i), dtype=torch.float64) * 50).to(dt)
        x[::97] *= 1e6
        out.append((f"f2x_{i}", x, bits, frac))
    return out


def gemm_cases():
    out = []
    specs = [(64, 512, 1024, torch.bfloat16, 32, False), (300, 264, 1096, torch.bfloat16, 64, True),
             (128, 384, 512, torch.float16, 32, True), (33, 520, 2048, torch.bfloat16, 64, False)]
    for i, (m, n, k, dt, bits, bias) in enumerate(specs):
        g = _g(200 + i)
        a = torch.randn(m, k, generator=g).to(dt)
        b = (0.05 * torch.randn(k, n, generator=g)).to(dt)
        bs = torch.randn(n, generator=g).to(dt) if bias else None
        out.append((f"gemm_{i}", a, b, bs, bits))
    return out


def attention_cases():
    out = []
    specs = [  # (seq_lens, q_lens, hq, hkv, d, page, dtype, int_bits, splits)
        ([300, 77, 1024], [1, 1, 1], 32, 8, 128, 16, torch.bfloat16, 32, 1),
        ([300, 77, 1024], [1, 1, 1], 32, 8, 128, 16, torch.bfloat16, 64, 4),
        ([130, 257], [130, 257], 8, 2, 64, 16, torch.float16, 32, 1),
        ([200, 64], [5, 64], 4, 2, 32, 16, torch.bfloat16, 32, 2),
        # the benchmark geometry (bf16, 32 query / 8 KV heads, head size 128, 16-token pages):
        ([80, 33], [80, 33], 32, 8, 128, 16, torch.bfloat16, 64, 1),        # prefill
        ([4500, 700, 64], [1, 1, 1], 32, 8, 128, 16, torch.bfloat16, 64, 8),  # long decode, 8 KV splits
        ([150], [150], 32, 8, 128, 16, torch.bfloat16, 64, 2),             # prefill through the split kernels
    ]
    for i, (sl, ql, hq, hkv, d, page, dt, bits, splits) in enumerate(specs):
        g = _g(300 + i)
        blocks = [-(-s // page) for s in sl]
        total = sum(blocks)
        kv = torch.randn(total + 1, 2, page, hkv, d, generator=g).to(dt)
        perm = torch.randperm(total, generator=g).to(torch.int32) + 1
        bt = torch.zeros(len(sl), max(blocks), dtype=torch.int32)
        o = 0
        for r, nb in enumerate(blocks):
            bt[r, :nb] = perm[o:o + nb]
            o += nb
        qsl = torch.zeros(len(ql) + 1, dtype=torch.int32)
        qsl[1:] = torch.tensor(ql, dtype=torch.int32).cumsum(0)
        q = torch.randn(int(qsl[-1]), hq, d, generator=g).to(dt)
        out.append((f"attn_{i}", q, kv, qsl, torch.tensor(sl, dtype=torch.int32), bt, max(ql), bits, splits))
    return out


def rms_cases():
    out = []
    for i, (rows, hidden, dt) in enumerate([(8, 4096, torch.float32), (5, 512, torch.bfloat16)]):
        g = _g(400 + i)
        x = torch.randn(rows, hidden, generator=g).to(dt)
        r = torch.randn(rows, hidden, generator=g).to(dt)
        w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dt)
        out.append((f"rms_{i}", x, r, w))
    return out


# Rows / heads of the integer accumulators that the fixture keeps (the full tensors would be
# several MB): the GEMM's first rows, and for attention these heads of every token.
GEMM_INT_ROWS = 32
ATTN_INT_HEADS = (0, 5, 31)
