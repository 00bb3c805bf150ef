"""Tensor-parallel row-parallel reduce on CPU ranks (gloo, world size 2 and 4):
the exchange step itself -- all_reduce(SUM) of integer accumulators followed by
one conversion -- gives the same bits as the unsharded GEMM.  The per-rank GEMM
is the CPU oracle here (the CUDA ops are injected the same way on GPUs)."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank: int, world: int, port: int, int_bits: int, out_dir: str) -> None:
    for p in (str(ROOT), str(ROOT / "vllm-triton-fixed-point-reductions_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fxpr_vllm import tp
        from oracle import fxp_oracle as orc

        g = torch.Generator().manual_seed(7)
        k_tile, K, M, N = 64, 64 * 8, 6, 10
        a = torch.randn(M, K, generator=g).to(torch.bfloat16)
        b = (0.05 * torch.randn(K, N, generator=g)).to(torch.bfloat16)
        bias = torch.randn(N, generator=g).to(torch.bfloat16)
        tp.check_shardable(K, world, k_tile)
        ks = K // world
        out = tp.row_parallel_gemm(
            a[:, rank * ks:(rank + 1) * ks], b[rank * ks:(rank + 1) * ks], bias, int_bits, 16,
            # accumulators in the width the GPU op returns (int16 is widened for the all-reduce)
            int_gemm=lambda x, w, ib, fb: orc._wrap_to_bits(
                orc.gemm_fxp(x, w, None, ib, fb, k_tile=k_tile, return_int=True), ib).to(
                    {16: torch.int16, 32: torch.int32, 64: torch.int64}[ib]),
            epilogue=lambda acc, bs, dt, fb: orc.gemm_epilogue(orc._wrap_to_bits(acc.to(torch.int64), int_bits), bs, dt, fb))
        full = orc.gemm_fxp(a, b, bias, int_bits, 16, k_tile=k_tile)
        assert torch.equal(out, full), f"rank {rank}: sharded result differs from the unsharded one"
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        assert all(torch.equal(gathered[0], t) for t in gathered)
        Path(out_dir, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,int_bits", [(2, 64), (4, 64), (2, 32), (2, 16)])
def test_row_parallel_integer_allreduce_matches_unsharded(world, int_bits, tmp_path):
    port = 29500 + (os.getpid() % 2000) + world
    mp.spawn(_worker, args=(world, port, int_bits, str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == [f"ok{r}" for r in range(world)]


def test_check_shardable_rejects_partial_tiles():
    for p in (str(ROOT), str(ROOT / "vllm-triton-fixed-point-reductions_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from fxpr_vllm import tp

    tp.check_shardable(4096, 8, 128)
    tp.check_shardable(14336, 8, 128)
    with pytest.raises(ValueError):
        tp.check_shardable(4096, 3, 64)
    with pytest.raises(ValueError):
        tp.check_shardable(4096 + 64, 8, 128)
