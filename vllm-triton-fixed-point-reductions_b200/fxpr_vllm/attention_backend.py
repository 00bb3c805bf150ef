"""The ``CUSTOM`` attention backend: vLLM's paged-KV attention layer on the
fixed-point kernel.

Keeps the contract of ``fxpr_vllm/attention_backend.py:41-277`` in the reference:
KV cache ``(num_blocks, 2, block_size, num_kv_heads, head_size)`` with identity
stride order, block sizes that are multiples of 16, head sizes >= 32,
FlashAttention's metadata and builder, decoder attention only, fp16/bf16 caches,
always causal, automatic KV-split choice, KV writes through vLLM's
``reshape_and_cache_flash``.  One deviation: when the caller's output buffer has
another dtype than the cache, the result is copied back into that buffer (the
reference writes it to a temporary only).
"""
from __future__ import annotations

import logging
from typing import ClassVar

import torch
from vllm.config.cache import CacheDType
from vllm.v1.attention.backend import (
    AttentionBackend,
    AttentionImpl,
    AttentionLayer,
    AttentionMetadata,
    AttentionMetadataBuilder,
    AttentionType,
    MultipleOf,
)

from . import _lib  # noqa: F401  (op registration)
from .config import get_runtime_config

logger = logging.getLogger("fxpr_vllm")

RCP_LN2 = 1.4426950408889634  # scores live in log2 space, so ALiBi slopes are pre-scaled

_SUPPORTED_KV_DTYPES = ("auto", "fp16", "bf16")


def _flash_classes() -> tuple[type[AttentionMetadata], type[AttentionMetadataBuilder]]:
    from vllm.v1.attention.backends.flash_attn import (
        FlashAttentionMetadata,
        FlashAttentionMetadataBuilder,
    )

    return FlashAttentionMetadata, FlashAttentionMetadataBuilder


def _as_int32(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.int32 else t.to(torch.int32)


class DeterministicAttentionBackend(AttentionBackend):
    accept_output_buffer: bool = True
    supported_dtypes: ClassVar[list[torch.dtype]] = [torch.float16, torch.bfloat16, torch.float32]
    supported_kv_cache_dtypes: ClassVar[list[CacheDType]] = ["auto", "float16", "bfloat16"]
    forward_includes_kv_cache_update: bool = False

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_supported_kernel_block_sizes() -> list[int | MultipleOf]:
        return [MultipleOf(16)]

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        if block_size % 16:
            raise ValueError("Block size must be a multiple of 16.")
        return (num_blocks, 2, block_size, num_kv_heads, head_size)

    @staticmethod
    def get_kv_cache_stride_order(include_num_layers_dimension: bool = False) -> tuple[int, ...]:
        return (1, 0, 2, 3, 4, 5) if include_num_layers_dimension else (0, 1, 2, 3, 4)

    @staticmethod
    def use_cascade_attention(*args, **kwargs) -> bool:
        return False

    @staticmethod
    def get_impl_cls() -> type["DeterministicAttentionImpl"]:
        return DeterministicAttentionImpl

    @staticmethod
    def get_metadata_cls() -> type[AttentionMetadata]:
        return _flash_classes()[0]

    @staticmethod
    def get_builder_cls() -> type[AttentionMetadataBuilder]:
        return _flash_classes()[1]

    @classmethod
    def supports_head_size(cls, head_size: int) -> bool:
        return head_size >= 32


class DeterministicAttentionImpl(AttentionImpl):
    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                 alibi_slopes: list[float] | None, sliding_window: int | None,
                 kv_cache_dtype: str = "auto", logits_soft_cap: float | None = None,
                 attn_type: AttentionType | None = AttentionType.DECODER,
                 *_extra_positional, **kwargs) -> None:
        if attn_type is not None and attn_type != AttentionType.DECODER:
            raise NotImplementedError(
                f"DeterministicAttention only supports decoder attention; got attn_type={attn_type!r}."
            )
        if kv_cache_dtype not in _SUPPORTED_KV_DTYPES:
            raise NotImplementedError(
                f"DeterministicAttention does not support kv_cache_dtype={kv_cache_dtype!r}; "
                f"supported: auto, fp16, bf16."
            )
        rt = get_runtime_config()
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = scale
        self.num_kv_heads = num_kv_heads
        self.num_kv_groups = num_heads // num_kv_heads
        self.kv_cache_dtype = kv_cache_dtype
        self.logits_soft_cap = float(logits_soft_cap) if logits_soft_cap else 0.0
        self.window_size = int(sliding_window) if sliding_window else 0
        self.attn_type = attn_type or AttentionType.DECODER
        self.fxp_int_bits = rt.fxp_int_bits
        self.fxp_frac_bits = rt.fxp_frac_bits
        self.alibi_slopes: torch.Tensor | None = None
        if alibi_slopes is not None:
            slopes = torch.tensor(alibi_slopes, dtype=torch.float32) * RCP_LN2
            assert slopes.shape == (num_heads,), (
                f"alibi_slopes shape {tuple(slopes.shape)} != (num_heads={num_heads},)")
            self.alibi_slopes = slopes

    def forward(self, layer: AttentionLayer, query: torch.Tensor, key: torch.Tensor,
                value: torch.Tensor, kv_cache: torch.Tensor,
                attn_metadata: AttentionMetadata | None, output: torch.Tensor | None = None,
                output_scale: torch.Tensor | None = None,
                output_block_scale: torch.Tensor | None = None, **kwargs) -> torch.Tensor:
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError(
                "DeterministicAttention does not support fp8/quantized output scales.")

        from .warmup import warmup_attention

        warmup_attention(self.num_heads, self.num_kv_heads, self.head_size, kv_cache.dtype,
                         query.device, self.window_size, self.logits_soft_cap,
                         self.fxp_int_bits, self.fxp_frac_bits)

        tokens = query.shape[0]
        flat = (tokens, self.num_heads * self.head_size)
        q = query.view(tokens, self.num_heads, self.head_size)
        if output is None:
            output = torch.empty_like(q)
        out = output.view(tokens, self.num_heads, self.head_size)

        if attn_metadata is None:          # vLLM's memory-profiling run
            out.zero_()
            return out.view(flat)

        if self.alibi_slopes is not None and self.alibi_slopes.device != q.device:
            self.alibi_slopes = self.alibi_slopes.to(q.device)

        # The launcher sizes its KV-split count and the decode kernel's score stash from the
        # block table's width, the only context bound the op's signature carries.  vLLM's table
        # is as wide as the model's maximum length; the metadata knows the longest live
        # sequence, so hand the kernel a view of just that many pages.
        block_table = attn_metadata.block_table
        max_seq_len = getattr(attn_metadata, "max_seq_len", None)
        if max_seq_len and block_table.dim() == 2:
            pages = -(-int(max_seq_len) // kv_cache.shape[2])
            if 0 < pages < block_table.shape[1]:
                block_table = block_table[:, :pages]

        q_in = q if q.dtype == kv_cache.dtype else q.to(kv_cache.dtype)
        o_in = out if out.dtype == q_in.dtype else torch.empty_like(out, dtype=q_in.dtype)
        torch.ops.fxpr.unified_attention_fxp(
            q_in, kv_cache, o_in,
            _as_int32(attn_metadata.query_start_loc), _as_int32(attn_metadata.seq_lens),
            block_table, int(attn_metadata.max_query_len), self.alibi_slopes,
            True, float(self.scale), int(self.fxp_int_bits), int(self.fxp_frac_bits),
            float(self.logits_soft_cap), int(self.window_size),
            0,  # let the launcher pick the KV-split count
        )
        if o_in is not out:
            out.copy_(o_in)
        return out.view(flat)

    def do_kv_cache_update(self, layer: AttentionLayer, key: torch.Tensor, value: torch.Tensor,
                           kv_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
        if self.attn_type in (AttentionType.ENCODER_ONLY, AttentionType.ENCODER):
            return
        from vllm._custom_ops import reshape_and_cache_flash

        k_cache, v_cache = kv_cache.unbind(1)
        reshape_and_cache_flash(key, value, k_cache, v_cache, slot_mapping, self.kv_cache_dtype,
                                layer._k_scale, layer._v_scale)
