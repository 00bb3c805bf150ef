"""Host-side logic that needs no GPU: the split policies (speed decisions only: every choice gives
the same bits) and the arg-max key arithmetic of the fused lm_head GEMM."""
from __future__ import annotations

import torch

import fxpr_vllm  # noqa: F401
from fxpr_vllm import _lib as L


def test_decode_gemm_split_policy_fills_the_sms_once():
    sms = 148
    for (n, k), want in {(4096, 4096): 4, (6144, 4096): 2, (28672, 4096): 1, (4096, 14336): 4,
                         (768, 4096): 8, (4096, 512): 1, (3584, 4096): 4, (4096, 1792): 4,
                         (128256, 4096): 1}.items():
        got = L.pick_split_k(64, n, k, 128, 64, sms)
        assert got == want, (n, k, got)
        tiles = -(-n // 128)
        assert got == 1 or tiles * got <= sms * 9 // 10          # clusters of whole-SM CTAs need headroom
        assert got == 1 or k // got >= 384
    assert L.pick_split_k(64, 4096, 4096, 128, 16, sms) == 1      # int16 accumulators never split
    assert L.pick_split_k(4096, 4096, 4096, 64, 64, sms) == 1     # the output tiles fill the GPU


def test_decode_attention_rank_policy():
    f = L.pick_num_splits_b200
    assert f(5, 64, 1, 32, 8, 8192, 148) == 5                     # an explicit request is kept
    assert f(64, 64, 1, 32, 8, 8192, 148) == 16                   # up to the cluster limit
    assert f(0, 64, 1, 32, 8, 8192, 148) == 8                     # long contexts: ~1024 keys per rank
    assert f(0, 64, 1, 32, 8, 4096, 148) == 4
    assert f(0, 64, 1, 32, 8, 1280, 148) == 1                     # the stash still leaves 4 CTAs per SM
    assert f(0, 64, 1, 32, 8, 1408, 148) == 2
    assert f(0, 64, 1, 16, 4, 1280, 148) == 2                     # fewer clusters: fill one wave
    assert f(0, 64, 1, 8, 2, 1280, 148) == 4
    assert f(0, 64, 1, 4, 1, 1280, 148) == 8
    assert f(0, 1, 1, 32, 8, 128, 148) == 1                       # two key tiles per rank at least
    assert f(0, 16, 4096, 32, 8, 4096, 148) == 1                  # prefill with enough row blocks


def test_argmax_keys_pick_the_first_maximum_and_combine_across_shards():
    g = torch.Generator().manual_seed(0)
    for dtype in (torch.bfloat16, torch.float16):
        x = torch.randn(7, 1000, generator=g).to(dtype)
        x[:, 900] = x[:, 17]                                      # ties (bf16 has plenty anyway)
        x[0, :] = -3.0                                            # a whole row of equal negatives
        x[1, 5] = float("inf")
        keys = L.argmax_keys_of(x)
        assert torch.equal(L.argmax_from_keys(keys), x.argmax(dim=-1))
        parts = [L.argmax_keys_of(x[:, a:b].contiguous(), n_offset=a) for a, b in ((0, 384), (384, 640), (640, 1000))]
        assert torch.equal(L.combine_argmax_keys(parts), keys)
        assert torch.equal(L.combine_argmax_keys(parts[::-1]), keys)   # order-free


def test_interleave_gate_up_layout():
    wg = torch.arange(12.0).reshape(3, 4)
    wu = -torch.arange(12.0).reshape(3, 4)
    p = L.interleave_gate_up(wg, wu)
    assert p.shape == (3, 8)
    assert torch.equal(p[:, 0::2], wg) and torch.equal(p[:, 1::2], wu)
