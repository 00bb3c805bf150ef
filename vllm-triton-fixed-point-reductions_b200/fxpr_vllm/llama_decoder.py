"""Random-init Llama-shaped decoder wired through the fixed-point ops, with tensor
parallelism whose only exchange is an integer all-reduce.

This is the workload of the fifth benchmark configuration (Llama-3-8B geometry, 64 decode
sequences, greedy sampling, TP = 1/2/4/8 with bit-identical logits), not a model zoo: no
checkpoint, no tokenizer, weights ~ N(0, 0.02) from a seeded generator.  Every reduction
runs in the integer domain: the GEMMs (``gemm_fxp`` / ``gemm_fxp_int``), the attention
(``unified_attention_fxp``), the norms (``rms_norm_fxp*``); RoPE, SiLU*mul and the KV-cache
write are element-wise torch ops.

Sharding follows vLLM's Llama (``vllm/model_executor/models/llama.py``): QKV and gate/up
column-parallel, attention heads split, o_proj and down_proj row-parallel, lm_head
vocab-parallel (all-gather), embedding and norms replicated.  A row-parallel layer keeps its
K-shard's integer accumulators, the group sums them (associative: any reduction order gives
the same bits), then one fixed->float epilogue runs on every rank.

``LocalGroup`` holds all shards in one process (single-GPU emulation used by the tests);
``DistGroup`` holds one shard per process and reduces with ``torch.distributed``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import library_ops as ops
from ._lib import (BLOCK_K_BY_DTYPE, argmax_from_keys, combine_argmax_keys, gemm_fxp_argmax, gemm_fxp_int_into,
                   gemm_silu_mul, interleave_gate_up, rope_kv_write, silu_mul_pairs, static_weights)
from .config import get_runtime_config
from .tp import check_shardable


@dataclass
class DecoderConfig:
    hidden: int = 4096
    ffn: int = 14336
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    vocab: int = 128256
    layers: int = 32
    dtype: torch.dtype = torch.bfloat16
    page: int = 16
    rope_theta: float = 500000.0
    eps: float = 1e-5
    int_bits: int = 64
    frac_bits: int = 16
    init_std: float = 0.02


class LocalGroup:
    """All ``size`` tensor-parallel shards live in this process (one GPU)."""

    def __init__(self, size: int):
        self.size = size
        self.local_ranks = list(range(size))

    def all_reduce_int(self, parts):
        total = parts[0].clone()
        for t in parts[1:]:
            total += t
        return [total] * len(parts)

    def all_gather_cols(self, parts):
        return torch.cat(parts, dim=-1)

    def all_gather_keys(self, parts):
        return list(parts)


class DistGroup:
    """One shard per process; ``torch.distributed`` carries the integer sums."""

    def __init__(self, group=None):
        self.group = group
        self.size = dist.get_world_size(group)
        self.local_ranks = [dist.get_rank(group)]
        # timing aid: with this set the exchanges are left out (results are then wrong, the
        # kernels and their shapes are unchanged), so a step's collective share can be measured
        self.skip_collectives = False

    def all_reduce_int(self, parts):
        if self.size > 1 and not self.skip_collectives:
            dist.all_reduce(parts[0], op=dist.ReduceOp.SUM, group=self.group)
        return parts

    def all_gather_cols(self, parts):
        if self.size == 1:
            return parts[0]
        if self.skip_collectives:
            return torch.cat([parts[0]] * self.size, dim=-1)
        out = [torch.empty_like(parts[0]) for _ in range(self.size)]
        dist.all_gather(out, parts[0].contiguous(), group=self.group)
        return torch.cat(out, dim=-1)

    def reduce_scatter_rows(self, acc):
        """Integer accumulators [T, H] of every rank -> this rank's T / size rows of their sum."""
        rows = acc.shape[0] // self.size
        r0 = dist.get_rank(self.group) * rows
        if self.skip_collectives:
            return acc[r0:r0 + rows].clone()
        out = torch.empty((rows, acc.shape[1]), device=acc.device, dtype=acc.dtype)
        dist.reduce_scatter_tensor(out, acc.contiguous(), op=dist.ReduceOp.SUM, group=self.group)
        return out

    def all_gather_rows(self, part):
        """This rank's rows -> all rows, in rank order."""
        out = torch.empty((part.shape[0] * self.size, part.shape[1]), device=part.device, dtype=part.dtype)
        if self.skip_collectives:
            out.view(self.size, *part.shape).copy_(part.unsqueeze(0).expand(self.size, *part.shape))
            return out
        dist.all_gather_into_tensor(out, part.contiguous(), group=self.group)
        return out

    def all_gather_keys(self, parts):
        """Arg-max keys of this rank's vocab shard -> every shard's keys (8 bytes per row)."""
        if self.size == 1 or self.skip_collectives:
            return list(parts) * (self.size if self.skip_collectives else 1)
        out = [torch.empty_like(parts[0]) for _ in range(self.size)]
        dist.all_gather(out, parts[0].contiguous(), group=self.group)
        return out


def _full_weight(shape, seed, device, dtype, std):
    g = torch.Generator(device=device).manual_seed(seed)
    return (std * torch.randn(shape, generator=g, device=device, dtype=torch.float32)).to(dtype)


class _Shard:
    """The weights and KV cache of one tensor-parallel rank."""

    def __init__(self):
        self.qkv = []
        self.o = []
        self.gate_up = []
        self.down = []
        self.lm_head = None
        self.kv_cache = []


class LlamaDecoder:
    def __init__(self, cfg: DecoderConfig, group, device, *, seed: int = 0, max_seqs: int = 64,
                 max_len: int = 1280, fused_elementwise: bool = True):
        self.cfg, self.group, self.device = cfg, group, torch.device(device)
        # fused CUDA kernels for RoPE + KV-cache write and SiLU*mul, or the same steps as torch ops
        self.fused = fused_elementwise
        # SiLU*mul inside the gate/up GEMM's epilogue for decode-sized batches (same bits as the
        # separate kernel); FXPR_DECODER_SILU_KERNEL=1 keeps the separate kernel (A/B timing)
        self.silu_epilogue = os.environ.get("FXPR_DECODER_SILU_KERNEL") != "1"
        # captured greedy decode steps take the next token from the lm_head GEMM's arg-max keys
        # instead of an argmax over the gathered logits; FXPR_DECODER_ARGMAX_KERNEL=1 keeps the latter
        self.greedy_fused = fused_elementwise and os.environ.get("FXPR_DECODER_ARGMAX_KERNEL") != "1"
        tp = group.size
        if cfg.q_heads % tp or cfg.kv_heads % tp or cfg.ffn % tp or cfg.vocab % tp:
            raise ValueError(f"tp={tp} does not divide the head / ffn / vocab sizes")
        k_tile = get_runtime_config().gemm_k_tile or BLOCK_K_BY_DTYPE[cfg.dtype]
        check_shardable(cfg.q_heads * cfg.head_dim, tp, k_tile)
        check_shardable(cfg.ffn, tp, k_tile)
        self.qh, self.kvh = cfg.q_heads // tp, cfg.kv_heads // tp
        hd, H = cfg.head_dim, cfg.hidden
        self.blocks_per_seq = -(-max_len // cfg.page)
        self.max_seqs = max_seqs
        self.shards = {r: _Shard() for r in group.local_ranks}
        dev, dt, std = self.device, cfg.dtype, cfg.init_std

        self.embed = _full_weight((cfg.vocab, H), seed * 1000 + 1, dev, dt, 1.0)
        self.norm_w = [torch.ones(H, device=dev, dtype=dt) for _ in range(2 * cfg.layers + 1)]
        for layer in range(cfg.layers):
            s0 = seed * 1000 + 10 * (layer + 1)
            # (K, N) row-major, the layout FixedPointLinearMethod keeps (quantisation_config.py)
            wq = _full_weight((H, cfg.q_heads * hd), s0 + 1, dev, dt, std)
            wk = _full_weight((H, cfg.kv_heads * hd), s0 + 2, dev, dt, std)
            wv = _full_weight((H, cfg.kv_heads * hd), s0 + 3, dev, dt, std)
            wo = _full_weight((cfg.q_heads * hd, H), s0 + 4, dev, dt, std)
            wg = _full_weight((H, cfg.ffn), s0 + 5, dev, dt, std)
            wu = _full_weight((H, cfg.ffn), s0 + 6, dev, dt, std)
            wd = _full_weight((cfg.ffn, H), s0 + 7, dev, dt, std)
            for r, sh in self.shards.items():
                q0, k0, f0 = r * self.qh * hd, r * self.kvh * hd, r * (cfg.ffn // tp)
                sh.qkv.append(torch.cat([wq[:, q0:q0 + self.qh * hd], wk[:, k0:k0 + self.kvh * hd],
                                         wv[:, k0:k0 + self.kvh * hd]], dim=1).contiguous())
                sh.o.append(wo[q0:q0 + self.qh * hd].contiguous())
                if self.fused:
                    # (gate_j, up_j) column pairs: the decode-shape GEMM applies SiLU*mul in its epilogue
                    sh.gate_up.append(interleave_gate_up(wg[:, f0:f0 + cfg.ffn // tp],
                                                         wu[:, f0:f0 + cfg.ffn // tp]))
                else:
                    sh.gate_up.append(torch.cat([wg[:, f0:f0 + cfg.ffn // tp],
                                                 wu[:, f0:f0 + cfg.ffn // tp]], dim=1).contiguous())
                sh.down.append(wd[f0:f0 + cfg.ffn // tp].contiguous())
                sh.kv_cache.append(torch.zeros((max_seqs * self.blocks_per_seq + 1, 2, cfg.page,
                                                self.kvh, hd), device=dev, dtype=dt))
            del wq, wk, wv, wo, wg, wu, wd
        wl = _full_weight((H, cfg.vocab), seed * 1000 + 2, dev, dt, std)
        vs = cfg.vocab // tp
        for r, sh in self.shards.items():
            sh.lm_head = wl[:, r * vs:(r + 1) * vs].contiguous()
        del wl
        # block 0 is left unused so that a zero block-table entry never aliases live data
        self.block_table = (torch.arange(max_seqs * self.blocks_per_seq, device=dev, dtype=torch.int32)
                            .reshape(max_seqs, self.blocks_per_seq) + 1)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd))
        ang = torch.arange(max_len, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.peer = None

    def enable_peer_reduce(self, max_rows: int | None = None) -> None:
        """Batches of at most ``max_rows`` tokens (decode steps) exchange through the
        peer-memory reduce + norm kernel instead of ``ncclAllReduce`` + a norm kernel.  Same
        bits; collective: every rank of the group must call it."""
        from .tp_fused import PeerReduceNorm

        if not isinstance(self.group, DistGroup) or self.group.size == 1:
            return
        c = self.cfg
        self.peer = PeerReduceNorm(max_rows or self.max_seqs, c.hidden, c.dtype, c.int_bits,
                                   group=self.group.group, device=self.device)

    # ------------------------------------------------------------------ pieces
    def _rope(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """Rotate-half RoPE in fp32 (element-wise, no reduction)."""
        half = self.cfg.head_dim // 2
        cos, sin = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        x1, x2 = x[..., :half].float(), x[..., half:].float()
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)

    def _write_kv(self, cache, k, v, seq_ids, pos):
        blk = self.block_table[seq_ids, pos // self.cfg.page].long()
        slot = pos % self.cfg.page
        cache[blk, 0, slot] = k
        cache[blk, 1, slot] = v

    def _row_parallel_norm(self, acts, weights, residual, norm_w):
        """Row-parallel GEMM, cross-rank integer sum, residual add and RMSNorm.  With more than one
        rank the conversion of the summed accumulators, the residual add and the norm are one
        kernel (same bits as the separate ones)."""
        c = self.cfg
        if self.group.size == 1:
            # nothing to exchange: the fused epilogue gives the same bits as int GEMM + epilogue
            x = ops.gemm_fxp(acts[0], weights[0], None, c.int_bits, c.frac_bits)
            return ops.rms_norm_fxp_residual(x, residual, norm_w, c.eps)
        rows = acts[0].shape[0]
        if self.peer is not None and rows <= self.peer.max_rows and not self.group.skip_collectives:
            # `residual` is the peer buffer's residual window (see forward)
            gemm_fxp_int_into(acts[0], weights[0], self.peer.acc[:rows], c.int_bits, c.frac_bits)
            # the residual only ever comes back into this call: each rank keeps its own rows current
            return self.peer.reduce_norm(rows, norm_w, None, c.eps, c.frac_bits, local_residual=True)
        accs = [ops.gemm_fxp_int(a, w, c.int_bits, c.frac_bits) for a, w in zip(acts, weights)]
        if isinstance(self.group, DistGroup) and rows >= 1024 and rows % self.group.size == 0:
            # Long batches (prefill): reduce-scatter by rows instead of all-reduce, residual add
            # and norm on this rank's rows only, all-gather of the normalised rows in the io
            # dtype.  The residual stays row-sharded for the whole forward pass (every exchange of
            # a pass takes this branch, and a rank only ever reads its own rows of it), so per
            # exchange 8 + 2 bytes per element cross the links instead of 16.  Same bits.
            part = self.group.reduce_scatter_rows(accs[0])
            r0 = self.group.local_ranks[0] * part.shape[0]
            y = ops.rms_norm_fxp_from_int(part, residual[r0:r0 + part.shape[0]], norm_w, None, c.eps, c.frac_bits)
            return self.group.all_gather_rows(y)
        accs = self.group.all_reduce_int(accs)
        return ops.rms_norm_fxp_from_int(accs[0], residual, norm_w, None, c.eps, c.frac_bits)

    # ------------------------------------------------------------------ forward
    def forward(self, tokens, seq_ids, pos, qsl, seq_lens, max_q: int, greedy_keys: bool = False):
        with static_weights():               # every GEMM operand b below is a weight of the model
            return self._forward(tokens, seq_ids, pos, qsl, seq_lens, max_q, greedy_keys)

    def _forward(self, tokens, seq_ids, pos, qsl, seq_lens, max_q: int, greedy_keys: bool = False):
        """tokens/seq_ids/pos: [T] (flattened batch); returns the logits of each sequence's
        last token, [B, vocab] in the io dtype, identical on every rank.  With ``greedy_keys``
        the lm_head GEMM also leaves each row's arg-max key (no pass over the logits, and with
        more than one rank only 8 bytes per row are exchanged): returns
        ``(this rank's [B, vocab / tp] logits shards, next tokens [B])``."""
        c = self.cfg
        T, hd = tokens.numel(), c.head_dim
        shards = [self.shards[r] for r in self.group.local_ranks]
        bt = self.block_table[: seq_lens.numel()]
        x = self.embed[tokens]
        if self.peer is not None and T <= self.peer.max_rows:
            residual = self.peer.residual[:T]       # every rank's copy is kept current by the kernel
            residual.copy_(x)
        else:
            residual = x.clone()
        h = ops.rms_norm_fxp(x, self.norm_w[0], c.eps)
        for layer in range(c.layers):
            outs = []
            for sh in shards:
                qkv = ops.gemm_fxp(h, sh.qkv[layer], None, c.int_bits, c.frac_bits)
                if self.fused:
                    q = rope_kv_write(qkv, self.cos, self.sin, pos, seq_ids, self.block_table,
                                      sh.kv_cache[layer], self.qh, self.kvh)
                else:
                    q, k, v = qkv.split([self.qh * hd, self.kvh * hd, self.kvh * hd], dim=1)
                    q = self._rope(q.reshape(T, self.qh, hd), pos)
                    k = self._rope(k.reshape(T, self.kvh, hd), pos)
                    self._write_kv(sh.kv_cache[layer], k, v.reshape(T, self.kvh, hd), seq_ids, pos)
                o = torch.empty_like(q)
                ops.unified_attention_fxp(q, sh.kv_cache[layer], o, qsl, seq_lens, bt, max_q, None, True,
                                          None, c.int_bits, c.frac_bits, 0.0, 0, 0)
                outs.append(o.reshape(T, self.qh * hd))
            h = self._row_parallel_norm(outs, [sh.o[layer] for sh in shards], residual, self.norm_w[2 * layer + 1])
            acts = []
            for sh in shards:
                if self.fused and self.silu_epilogue:
                    acts.append(gemm_silu_mul(h, sh.gate_up[layer], c.int_bits, c.frac_bits))
                elif self.fused:
                    acts.append(silu_mul_pairs(ops.gemm_fxp(h, sh.gate_up[layer], None, c.int_bits, c.frac_bits)))
                else:
                    gu = ops.gemm_fxp(h, sh.gate_up[layer], None, c.int_bits, c.frac_bits)
                    f = gu.shape[1] // 2
                    acts.append((torch.nn.functional.silu(gu[:, :f].float()) * gu[:, f:].float()).to(c.dtype))
            # the norm in front of the next layer (or, after the last layer, the final norm)
            h = self._row_parallel_norm(acts, [sh.down[layer] for sh in shards], residual,
                                        self.norm_w[2 * layer + 2])
        last = h[(qsl[1:] - 1).long()]
        if greedy_keys:
            vs = c.vocab // self.group.size
            both = [gemm_fxp_argmax(last, self.shards[r].lm_head, None, c.int_bits, c.frac_bits, n_offset=r * vs)
                    for r in self.group.local_ranks]
            keys = combine_argmax_keys(self.group.all_gather_keys([k for _, k in both]))
            return [lg for lg, _ in both], argmax_from_keys(keys)
        parts = [ops.gemm_fxp(last, sh.lm_head, None, c.int_bits, c.frac_bits) for sh in shards]
        return self.group.all_gather_cols(parts)

    # ------------------------------------------------------------------ generation
    def prefill(self, prompts: torch.Tensor) -> torch.Tensor:
        """prompts [B, L] int64 -> logits [B, vocab] of the last prompt token."""
        B, L = prompts.shape
        dev = self.device
        seq_ids = torch.arange(B, device=dev).repeat_interleave(L)
        pos = torch.arange(L, device=dev).repeat(B)
        qsl = torch.arange(B + 1, device=dev, dtype=torch.int32) * L
        seq_lens = torch.full((B,), L, device=dev, dtype=torch.int32)
        return self.forward(prompts.reshape(-1), seq_ids, pos, qsl, seq_lens, L)

    def decode_step(self, tokens: torch.Tensor, cur_len: int) -> torch.Tensor:
        """tokens [B] are appended at position ``cur_len`` of every sequence."""
        B = tokens.numel()
        dev = self.device
        seq_ids = torch.arange(B, device=dev)
        pos = torch.full((B,), cur_len, device=dev, dtype=torch.long)
        qsl = torch.arange(B + 1, device=dev, dtype=torch.int32)
        seq_lens = torch.full((B,), cur_len + 1, device=dev, dtype=torch.int32)
        return self.forward(tokens, seq_ids, pos, qsl, seq_lens, 1)

    @staticmethod
    def greedy(logits: torch.Tensor) -> torch.Tensor:
        return logits.argmax(dim=-1)        # exact in the io dtype: no float copy of [B, vocab]

    # ------------------------------------------------------------------ CUDA-graph decode
    def capture_decode(self, first_tokens: torch.Tensor, start_len: int):
        """Capture one greedy decode step (forward + argmax + position update) in a CUDA
        graph; ``replay_decode()`` then runs a step with a single launch.  Positions, lengths
        and the current tokens live in device tensors that the graph itself advances."""
        B, dev = first_tokens.numel(), self.device
        self._g_tok = first_tokens.clone()
        self._g_pos = torch.full((B,), start_len, device=dev, dtype=torch.long)
        self._g_lens = torch.full((B,), start_len + 1, device=dev, dtype=torch.int32)
        self._g_ids = torch.arange(B, device=dev)
        self._g_qsl = torch.arange(B + 1, device=dev, dtype=torch.int32)

        def step():
            if self.greedy_fused:
                return self.forward(self._g_tok, self._g_ids, self._g_pos, self._g_qsl, self._g_lens, 1,
                                    greedy_keys=True)
            logits = self.forward(self._g_tok, self._g_ids, self._g_pos, self._g_qsl, self._g_lens, 1)
            return logits, self.greedy(logits)

        # eager warm-up on a side stream (allocations, split-K scratch, module state); it
        # writes the KV slot at start_len, which the first replay overwrites with the same data
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._g_logits, tok = step()
            self._g_tok.copy_(tok)
            self._g_pos += 1
            self._g_lens += 1

    def replay_decode(self):
        """One captured decode step; returns the logits buffer (overwritten by the next replay):
        the full ``[B, vocab]`` tensor, or with ``greedy_fused`` this rank's vocab shards (see
        ``last_logits``)."""
        self._graph.replay()
        return self._g_logits

    def last_logits(self) -> torch.Tensor:
        """The ``[B, vocab]`` logits of the last replayed step on every rank (with ``greedy_fused``
        the shards are gathered here, outside the step)."""
        if self.greedy_fused:
            return self.group.all_gather_cols(list(self._g_logits))
        return self._g_logits
