"""The peer-memory reduce + residual + RMSNorm kernel (``fxpr_tp_reduce_norm``).

One GPU: a group of one rank against ``rms_norm_fxp_from_int`` (same bits), and a wait that
runs out (a second rank whose flags nothing ever sets) reported through the status word with
the context still usable.  Two GPUs (skipped on smaller boxes): two processes, one per GPU,
against the integer all-reduce + ``rms_norm_fxp_from_int``, repeated calls and a CUDA graph.
"""
from __future__ import annotations

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

import fxpr_vllm  # noqa: F401
from fxpr_vllm import _lib as L

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("int_bits", [32, 64])
@pytest.mark.parametrize("rows,hidden,use_bias", [(1, 4096, False), (7, 1000, True), (64, 4096, True),
                                                  (33, 8192, False)])
def test_one_rank_equals_from_int_kernel(dtype, int_bits, rows, hidden, use_bias):
    from fxpr_vllm.tp_fused import PeerReduceNorm

    g = torch.Generator().manual_seed(rows + hidden)
    idt = torch.int32 if int_bits == 32 else torch.int64
    pr = PeerReduceNorm(64, hidden, dtype, int_bits, device="cuda:0")
    try:
        w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).cuda()
        bias = torch.randn(hidden, generator=g).to(dtype).cuda() if use_bias else None
        res = torch.randn(rows, hidden, generator=g).to(dtype).cuda()
        pr.residual[:rows].copy_(res)
        for _ in range(3):                  # the residual carries over from call to call
            acc = (torch.randn(rows, hidden, generator=g) * 3 * 65536).to(idt).cuda()
            pr.acc[:rows].copy_(acc)
            want = torch.ops.fxpr.rms_norm_fxp_from_int(acc, res, w, bias, 1e-6, 16)
            got = pr.reduce_norm(rows, w, bias, 1e-6, 16)
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
            assert torch.equal(pr.residual[:rows].view(torch.uint8), res.view(torch.uint8))
        L.check_device_status()
    finally:
        pr.close()


def test_wait_that_runs_out_sets_the_status_word():
    """Rank 0 of a two-rank group whose second rank never runs: the ready flag never arrives,
    the kernel gives up after the given number of clocks, reports FXPR_ERR_TIMEOUT and leaves
    the peer's buffers alone; the context stays usable."""
    from fxpr_vllm.tp_fused import PeerReduceNorm

    L.check_device_status()
    pr = PeerReduceNorm(8, 256, torch.bfloat16, 64, device="cuda:0", timeout_cycles=2_000_000,
                        _fake_world=2)
    try:
        w = torch.ones(256, dtype=torch.bfloat16, device="cuda")
        pr.acc.fill_(65536)
        y_before = pr.y.clone()
        pr.reduce_norm(8, w, None, 1e-6, 16)
        with pytest.raises(RuntimeError, match="(?i)time"):
            L.check_device_status()
        assert torch.equal(pr.y, y_before)                     # nothing was written
        assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
        L.check_device_status()                                # the word was cleared
    finally:
        pr.close()


_WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, {root!r}); sys.path.insert(0, {pkg!r})
    import torch, torch.distributed as dist
    import fxpr_vllm
    from fxpr_vllm import _lib as L
    from fxpr_vllm.tp_fused import PeerReduceNorm
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    rows, hidden = 64, 4096
    pr = PeerReduceNorm(rows, hidden, torch.bfloat16, 64, device=dev)
    g = torch.Generator().manual_seed(1)                     # same residual and weight everywhere
    res0 = torch.randn(rows, hidden, generator=g).to(torch.bfloat16).to(dev)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(dev)
    gr = torch.Generator().manual_seed(100 + rank)           # per-rank accumulators
    ok = True
    for n in (64, 5, 1, 64):
        res = res0[:n].clone()
        pr.residual[:n].copy_(res)
        for it in range(4):
            acc = (torch.randn(n, hidden, generator=gr) * 3 * 65536).to(torch.int64).to(dev)
            pr.acc[:n].copy_(acc)
            tot = acc.clone()
            dist.all_reduce(tot)
            want = torch.ops.fxpr.rms_norm_fxp_from_int(tot, res, w, None, 1e-6, 16)
            got = pr.reduce_norm(n, w, None, 1e-6, 16)
            ok &= bool(torch.equal(got, want)) and bool(torch.equal(pr.residual[:n], res))
    # row-sharded residual: a rank keeps only its own rows of its residual copy current
    n = 64
    res = res0.clone()
    pr.residual[:n].copy_(res)
    per = -(-n // world)
    lo, hi = rank * per, min(n, (rank + 1) * per)
    for it in range(3):
        acc = (torch.randn(n, hidden, generator=gr) * 3 * 65536).to(torch.int64).to(dev)
        pr.acc[:n].copy_(acc)
        tot = acc.clone()
        dist.all_reduce(tot)
        want = torch.ops.fxpr.rms_norm_fxp_from_int(tot, res, w, None, 1e-6, 16)
        got = pr.reduce_norm(n, w, None, 1e-6, 16, local_residual=True)
        ok &= bool(torch.equal(got, want)) and bool(torch.equal(pr.residual[lo:hi], res[lo:hi]))
    # replayed from a CUDA graph: the call counter lives on the device
    pr.residual[:rows].copy_(res0)
    acc = (torch.randn(rows, hidden, generator=gr) * 3 * 65536).to(torch.int64).to(dev)
    pr.acc[:rows].copy_(acc)
    tot = acc.clone(); dist.all_reduce(tot)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        pr.reduce_norm(rows, w, None, 1e-6, 16)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = pr.reduce_norm(rows, w, None, 1e-6, 16)
    res = res0.clone()
    pr.residual[:rows].copy_(res0)
    for it in range(5):
        want = torch.ops.fxpr.rms_norm_fxp_from_int(tot, res, w, None, 1e-6, 16)
        graph.replay()
        ok &= bool(torch.equal(out, want)) and bool(torch.equal(pr.residual[:rows], res))
    L.check_device_status()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    pr.close()
    dist.destroy_process_group()
    if rank == 0:
        print("PEER_REDUCE_OK" if int(flag.item()) == 1 else "PEER_REDUCE_MISMATCH")
""")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_equal_all_reduce_then_from_int(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=str(ROOT), pkg=str(ROOT / "vllm-triton-fixed-point-reductions_b200")))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "PEER_REDUCE_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
