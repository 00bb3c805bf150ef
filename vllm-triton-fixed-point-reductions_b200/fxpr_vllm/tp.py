"""Tensor-parallel row-parallel linear with an integer all-reduce.

vLLM reduces the bf16 outputs of a row-parallel layer across ranks with a float
all-reduce (``vllm/model_executor/layers/linear.py``, after ``quant_method.apply``),
whose result depends on the number of ranks.  Here each rank keeps the *integer*
accumulators of its K-shard, the ranks sum integers (associative, so any
reduction tree gives the same bits), and every rank converts once and adds the
bias.  With K/tp a whole number of K-tiles the union of the ranks' K-tiles is
the TP=1 tile set, hence bit-identical outputs for TP = 1/2/4/8.  The reference
has no counterpart.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import library_ops as ops


def check_shardable(k_total: int, tp: int, k_tile: int) -> None:
    if k_total % tp or (k_total // tp) % k_tile:
        raise ValueError(
            f"row-parallel K={k_total} over tp={tp} must give whole K-tiles of {k_tile} per rank"
        )


def row_parallel_gemm(x_shard: torch.Tensor, w_shard: torch.Tensor, bias: torch.Tensor | None,
                      fxp_int_bits: int, fxp_frac_bits: int, group=None,
                      int_gemm=None, epilogue=None) -> torch.Tensor:
    """``x_shard [M, K/tp] @ w_shard [K/tp, N]`` summed over the group in integers.

    ``int_gemm`` / ``epilogue`` default to the CUDA ops; tests on CPU ranks inject
    the oracle's functions to exercise the exchange itself.
    """
    int_gemm = int_gemm or ops.gemm_fxp_int
    epilogue = epilogue or ops.gemm_fxp_epilogue
    acc = int_gemm(x_shard, w_shard, fxp_int_bits, fxp_frac_bits)
    if group is not None or (dist.is_available() and dist.is_initialized()):
        if dist.get_world_size(group) > 1:
            if acc.dtype == torch.int16:
                # NCCL has no 16-bit integer sum: reduce in int32 and wrap back to 16 bits,
                # which equals a 16-bit wrap-around sum of the ranks' accumulators
                wide = acc.to(torch.int32)
                dist.all_reduce(wide, op=dist.ReduceOp.SUM, group=group)
                acc = wide.to(torch.int16)
            else:
                dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=group)
    return epilogue(acc, bias, x_shard.dtype, fxp_frac_bits)
