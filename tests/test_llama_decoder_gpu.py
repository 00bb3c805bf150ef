"""The decoder of the fifth benchmark configuration at a reduced size: logits must be
bit-identical for tensor-parallel degrees 1/2/4 (all shards emulated on one GPU; the
exchange is the integer sum of the row-parallel accumulators)."""
from __future__ import annotations

import pytest
import torch

import fxpr_vllm  # noqa: F401
from fxpr_vllm.llama_decoder import DecoderConfig, LlamaDecoder, LocalGroup

pytestmark = pytest.mark.gpu


def _run(tp, int_bits):
    cfg = DecoderConfig(hidden=512, ffn=1024, q_heads=8, kv_heads=4, head_dim=64, vocab=1024, layers=2,
                        int_bits=int_bits)
    m = LlamaDecoder(cfg, LocalGroup(tp), "cuda", seed=3, max_seqs=5, max_len=96)
    g = torch.Generator().manual_seed(11)
    prompts = torch.randint(0, cfg.vocab, (5, 40), generator=g).cuda()
    outs = [m.prefill(prompts)]
    tok = m.greedy(outs[-1])
    for step in range(3):
        outs.append(m.decode_step(tok, 40 + step))
        tok = m.greedy(outs[-1])
    return torch.stack(outs), tok


@pytest.mark.parametrize("int_bits", [64, 32])
def test_logits_bit_identical_across_tp(int_bits):
    ref, tok = _run(1, int_bits)
    assert torch.isfinite(ref.float()).all()
    assert ref.float().abs().max() > 0
    for tp in (2, 4):
        got, tok2 = _run(tp, int_bits)
        assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), f"tp={tp}"
        assert torch.equal(tok, tok2)


def test_decode_matches_prefill_of_the_longer_prompt():
    """Batch invariance through the whole stack: the logits after prefill(40) + one decoded
    token equal the logits of prefill(41) on the extended prompt."""
    cfg = DecoderConfig(hidden=512, ffn=1024, q_heads=8, kv_heads=4, head_dim=64, vocab=1024, layers=2)
    g = torch.Generator().manual_seed(12)
    prompts = torch.randint(0, cfg.vocab, (3, 41), generator=g).cuda()
    a = LlamaDecoder(cfg, LocalGroup(1), "cuda", seed=3, max_seqs=3, max_len=96)
    a.prefill(prompts[:, :40].contiguous())
    la = a.decode_step(prompts[:, 40].contiguous(), 40)
    b = LlamaDecoder(cfg, LocalGroup(1), "cuda", seed=3, max_seqs=3, max_len=96)
    lb = b.prefill(prompts)
    assert torch.equal(la.view(torch.int16), lb.view(torch.int16))


def test_graph_decode_equals_eager_decode():
    cfg = DecoderConfig(hidden=512, ffn=1024, q_heads=8, kv_heads=4, head_dim=64, vocab=1024, layers=2)
    g = torch.Generator().manual_seed(13)
    prompts = torch.randint(0, cfg.vocab, (4, 33), generator=g).cuda()
    a = LlamaDecoder(cfg, LocalGroup(2), "cuda", seed=5, max_seqs=4, max_len=64)
    tok = a.greedy(a.prefill(prompts))
    eager = []
    t = tok
    for step in range(4):
        eager.append(a.decode_step(t, 33 + step))
        t = a.greedy(eager[-1])
    b = LlamaDecoder(cfg, LocalGroup(2), "cuda", seed=5, max_seqs=4, max_len=64)
    tok_b = b.greedy(b.prefill(prompts))
    assert torch.equal(tok, tok_b)
    b.capture_decode(tok_b, 33)
    for step in range(4):
        b.replay_decode()
        got = b.last_logits().clone()
        assert torch.equal(got.view(torch.int16), eager[step].view(torch.int16)), step


def test_fused_rope_kv_write_equals_torch_path():
    """The fused RoPE + KV-cache-write kernel against the same steps as torch ops: rotated Q and
    the cache contents must agree bit for bit (separate multiply / subtract roundings on both
    sides)."""
    from fxpr_vllm._lib import rope_kv_write, silu_mul
    cfg = DecoderConfig(hidden=512, ffn=1024, q_heads=8, kv_heads=4, head_dim=64, vocab=1024, layers=1)
    m = LlamaDecoder(cfg, LocalGroup(1), "cuda", seed=3, max_seqs=3, max_len=96, fused_elementwise=False)
    g = torch.Generator(device="cuda").manual_seed(5)
    T = 3 * 37
    qkv = torch.randn((T, (8 + 2 * 4) * 64), generator=g, device="cuda").to(cfg.dtype)
    seq_ids = torch.arange(3, device="cuda").repeat_interleave(37)
    pos = torch.arange(37, device="cuda").repeat(3) + 5
    cache_a = m.shards[0].kv_cache[0]
    cache_b = torch.zeros_like(cache_a)
    q, k, v = qkv.split([8 * 64, 4 * 64, 4 * 64], dim=1)
    q_ref = m._rope(q.reshape(T, 8, 64), pos)
    m._write_kv(cache_a, m._rope(k.reshape(T, 4, 64), pos), v.reshape(T, 4, 64), seq_ids, pos)
    q_got = rope_kv_write(qkv, m.cos, m.sin, pos, seq_ids, m.block_table, cache_b, 8, 4)
    assert torch.equal(q_got.view(torch.int16), q_ref.view(torch.int16))
    assert torch.equal(cache_b.view(torch.int16), cache_a.view(torch.int16))
    gu = torch.randn((50, 2 * 1024), generator=g, device="cuda").to(cfg.dtype)
    ref = (torch.nn.functional.silu(gu[:, :1024].float()) * gu[:, 1024:].float())
    got = silu_mul(gu).float()
    assert (got - ref).abs().max() <= 0.01 * ref.abs().max()
