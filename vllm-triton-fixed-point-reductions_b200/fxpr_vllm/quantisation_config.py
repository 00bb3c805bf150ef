"""The ``fixedpoint`` quantization config: every linear layer (and the lm_head)
runs through ``gemm_fxp``.

Same names and behaviour as ``fxpr_vllm/quantisation_config.py:25-188`` of the
reference: ``FixedPointConfig`` (name ``fixedpoint``, fp16/bf16/fp32 activations,
no config files), ``FixedPointLinearMethod`` (weight stored ``(out, in)``, turned
once into the ``(K, N)`` ``weight_native`` the GEMM wants) and
``FixedPointEmbeddingMethod`` (lookups stay on ``F.embedding``; only the lm_head
matmul is fixed-point, opt out with ``FXPR_DISABLE_LM_HEAD=1``).

Addition: a row-parallel layer with ``reduce_results`` does its cross-rank sum on
the integer accumulators inside ``apply`` (see ``tp.py``) and switches vLLM's
float all-reduce off, which is what makes TP=1/2/4/8 bit-identical.
"""
from __future__ import annotations

import logging
from collections.abc import Sequence
from typing import Any

import torch
import torch.nn as nn
from vllm.model_executor.layers.linear import LinearBase
from vllm.model_executor.layers.quantization.base_config import (
    QuantizationConfig,
    QuantizeMethodBase,
)
from vllm.model_executor.layers.vocab_parallel_embedding import VocabParallelEmbedding
from vllm.model_executor.parameter import ModelWeightParameter
from vllm.model_executor.utils import set_weight_attrs

from .config import get_runtime_config
from .library_ops import gemm_fxp
from .warmup import warmup_gemm, warmup_rms_norm

logger = logging.getLogger("fxpr_vllm")


def _to_kn(weight: torch.Tensor) -> torch.Tensor:
    """(out, in) checkpoint layout -> contiguous (K, N) = (in, out)."""
    with torch.no_grad():
        return weight.data.t().contiguous()


class _FxpMethodBase(QuantizeMethodBase):
    def __init__(self, config: "FixedPointConfig") -> None:
        self.config = config
        rt = get_runtime_config()
        self.fxp_int_bits = rt.fxp_int_bits
        self.fxp_frac_bits = rt.fxp_frac_bits

    def _matmul(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        from ._lib import static_weights

        with static_weights():               # weight_native is a loaded weight, never a kernel's fresh output
            return gemm_fxp(x, layer.weight_native, bias, self.fxp_int_bits, self.fxp_frac_bits)


class FixedPointLinearMethod(_FxpMethodBase):
    def create_weights(self, layer: nn.Module, input_size_per_partition: int,
                       output_partition_sizes: Sequence[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype, **extra_weight_attrs: Any) -> None:
        loader = extra_weight_attrs.pop("weight_loader")
        shape = (sum(output_partition_sizes), input_size_per_partition)
        weight = ModelWeightParameter(data=torch.empty(shape, dtype=params_dtype), input_dim=1,
                                      output_dim=0, weight_loader=loader)
        layer.register_parameter("weight", weight)
        set_weight_attrs(weight, extra_weight_attrs)

    def process_weights_after_loading(self, layer: nn.Module) -> None:
        layer.weight_native = _to_kn(layer.weight)
        del layer.weight
        layer.register_parameter("weight", None)
        self._setup_tp(layer)
        warmup_gemm(layer.weight_native, self.fxp_int_bits, self.fxp_frac_bits)
        warmup_rms_norm(layer.weight_native.shape[0], layer.weight_native.dtype,
                        layer.weight_native.device)

    def _setup_tp(self, layer: nn.Module) -> None:
        """Row-parallel layers that vLLM would all-reduce in floating point are reduced
        here in integers instead (bias is then added after the reduce on every rank).

        The integer reduce only gives TP-independent bits when every rank's K-shard is a
        whole number of K-tiles (the union of the shards' tiles is then the TP=1 tile
        set); a layer that does not shard that way keeps vLLM's float all-reduce, with a
        warning, rather than silently producing TP-dependent results."""
        layer._fxp_int_reduce = False
        try:
            from vllm.model_executor.layers.linear import RowParallelLinear
        except Exception:
            return
        tp = getattr(layer, "tp_size", 1)
        if isinstance(layer, RowParallelLinear) and tp > 1 and getattr(layer, "reduce_results", False):
            from ._lib import BLOCK_K_BY_DTYPE
            from .tp import check_shardable

            k_tile = get_runtime_config().gemm_k_tile or BLOCK_K_BY_DTYPE[layer.weight_native.dtype]
            k_total = getattr(layer, "input_size", layer.weight_native.shape[0] * tp)
            try:
                check_shardable(int(k_total), int(tp), int(k_tile))
            except ValueError as exc:
                logger.warning("fxpr_vllm: %s; this layer keeps vLLM's float all-reduce and its "
                               "bits depend on the TP degree", exc)
                return
            layer._fxp_int_reduce = True
            layer.reduce_results = False

    def apply(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if getattr(layer, "_fxp_int_reduce", False):
            from vllm.distributed import get_tp_group

            from .tp import row_parallel_gemm

            lead = x.shape[:-1]
            out = row_parallel_gemm(x.reshape(-1, x.shape[-1]), layer.weight_native,
                                    getattr(layer, "bias", None) if not layer.skip_bias_add else None,
                                    self.fxp_int_bits, self.fxp_frac_bits,
                                    group=get_tp_group().device_group)
            return out.reshape(*lead, out.shape[-1])
        return self._matmul(layer, x, bias)


class FixedPointEmbeddingMethod(_FxpMethodBase):
    """For VocabParallelEmbedding / ParallelLMHead: ``weight`` stays for the lookup,
    ``weight_native`` is its transpose for the lm_head matmul."""

    def create_weights(self, layer: nn.Module, input_size_per_partition: int,
                       output_partition_sizes: Sequence[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype, **extra_weight_attrs: Any) -> None:
        shape = (sum(output_partition_sizes), input_size_per_partition)
        weight = nn.Parameter(torch.empty(shape, dtype=params_dtype), requires_grad=False)
        set_weight_attrs(weight, {"input_dim": 1, "output_dim": 0})
        layer.register_parameter("weight", weight)
        set_weight_attrs(weight, extra_weight_attrs)

    def process_weights_after_loading(self, layer: nn.Module) -> None:
        layer.weight_native = _to_kn(layer.weight)
        warmup_gemm(layer.weight_native, self.fxp_int_bits, self.fxp_frac_bits)

    def apply(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        return self._matmul(layer, x, bias)

    def embedding(self, layer: nn.Module, input_: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.embedding(input_, layer.weight)


class FixedPointConfig(QuantizationConfig):
    def __init__(self) -> None:
        pass

    def __repr__(self) -> str:
        return "FixedPointConfig()"

    @classmethod
    def get_name(cls) -> str:
        return "fixedpoint"

    @classmethod
    def get_supported_act_dtypes(cls) -> list[torch.dtype]:
        return [torch.float16, torch.bfloat16, torch.float32]

    @classmethod
    def get_min_capability(cls) -> int:
        return 100  # the kernels are sm_100a only

    @classmethod
    def get_config_filenames(cls) -> list[str]:
        return []

    @classmethod
    def from_config(cls, config: dict[str, Any]) -> "FixedPointConfig":
        return cls()

    def get_quant_method(self, layer: nn.Module, prefix: str) -> QuantizeMethodBase | None:
        if isinstance(layer, LinearBase):
            return FixedPointLinearMethod(self)
        if isinstance(layer, VocabParallelEmbedding) and get_runtime_config().enable_lm_head:
            return FixedPointEmbeddingMethod(self)
        return None

    def get_scaled_act_names(self) -> list[str]:
        return []
