"""The CPU oracle against the reference's own known-answer vectors, plus the
oracle's internal invariants (order-freedom, sharding).  No GPU needed."""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import fxp_oracle as orc

GOLD = json.loads((Path(__file__).parent / "golden" / "cast_known_answers.json").read_text())


@pytest.mark.parametrize("case", GOLD["float_to_fixed"])
def test_float_to_fixed_known_values(case):
    x = torch.tensor(case["x"], dtype=torch.float32)
    q = orc.float_to_fixed(x, case["int_bits"], case["frac_bits"])
    assert q.tolist() == case["q"]


@pytest.mark.parametrize("case", GOLD["saturation"])
def test_saturation_bounds(case):
    x = torch.tensor(case["x"], dtype=torch.float32)
    q = orc.float_to_fixed(x, case["int_bits"], case["frac_bits"]).tolist()
    for got, lo, hi in zip(q, case["q_low"], case["q_high"]):
        assert lo <= got <= hi
    # cvt.rni.sat gives the exact limits
    assert q[0] == 2**31 - 1 and q[1] == -(2**31)


@pytest.mark.parametrize("case", GOLD["float_roundtrip_exact"])
def test_float_roundtrip_exact(case):
    x = torch.tensor(case["x"], dtype=torch.float32)
    q = orc.float_to_fixed(x, case["int_bits"], case["frac_bits"])
    back = orc.fixed_to_float(q, 32, case["frac_bits"])
    assert torch.equal(back, x)


@pytest.mark.parametrize("case", GOLD["float_roundtrip_half_step"])
def test_float_roundtrip_half_step(case):
    x = torch.tensor(case["x"], dtype=torch.float32)
    step = 2.0 ** -case["frac_bits"]
    back = orc.fixed_to_float(orc.float_to_fixed(x, case["int_bits"], case["frac_bits"]), 32,
                              case["frac_bits"])
    assert torch.all((x - back).abs() <= step / 2 + 1e-7)
    assert torch.any(x != back)


@pytest.mark.parametrize("case", GOLD["fixed_roundtrip_exact"])
def test_fixed_roundtrip_exact(case):
    q = torch.tensor(case["q"], dtype=torch.int32)
    f = orc.fixed_to_float(q, 32, case["frac_bits"])
    assert torch.equal(orc.float_to_fixed(f, case["int_bits"], case["frac_bits"]), q)


@pytest.mark.parametrize("case", GOLD["sum_on_grid"])
def test_sum_on_grid_matches_float_sum(case):
    q = torch.tensor(case["q"], dtype=torch.int32)
    x = orc.fixed_to_float(q.to(torch.int64), 32, case["frac_bits"])
    assert torch.equal(orc.float_to_fixed(x, 32, case["frac_bits"]), q)
    fixed = orc.fixed_to_float(orc.float_to_fixed(x, 32, 16).sum().reshape(1), 32, 16)
    assert fixed.view(torch.int32).item() == x.sum(dtype=torch.float32).reshape(1).view(torch.int32).item()


@pytest.mark.parametrize("case", GOLD["sum_saturates"])
def test_sum_saturates(case):
    x = torch.tensor(case["x"], dtype=torch.float32)
    s = orc.float_to_fixed(x, case["int_bits"], case["frac_bits"]).to(torch.int64).sum()
    assert int(s.clamp(-(2**31), 2**31 - 1)) == case["clamped_sum"]


@pytest.mark.parametrize("case", GOLD["associativity"])
def test_fixed_sum_is_order_free(case):
    outs = []
    for order in (case["order_a"], case["order_b"]):
        q = orc.float_to_fixed(torch.tensor(order, dtype=torch.float32), 64, 16)
        acc = torch.zeros((), dtype=torch.int64)
        for v in q:
            acc = acc + v
        outs.append(orc.fixed_to_float(acc.reshape(1), 32, 16).item())
    assert outs[0] == outs[1] == case["sum"]


def test_nan_and_int16_and_int64_edges():
    x = torch.tensor([float("nan"), 1e30, -1e30, 0.5, 2.5e-5, 0.49999], dtype=torch.float32)
    assert orc.float_to_fixed(x, 32, 16).tolist()[:3] == [0, 2**31 - 1, -(2**31)]
    assert orc.float_to_fixed(x, 16, 8).tolist()[:4] == [0, 32767, -32768, 128]
    q64 = orc.float_to_fixed(x, 64, 32).tolist()
    assert q64[0] == -(2**63) and q64[1] == 2**63 - 1 and q64[2] == -(2**63)
    # half-to-even ties
    t = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5], dtype=torch.float32) / 65536.0
    assert orc.float_to_fixed(t, 32, 16).tolist() == [0, 2, 2, 0, -2]


def test_exp2_det_accuracy_and_edges():
    t = torch.linspace(-60.0, 0.0, 20001, dtype=torch.float32)
    got = orc.exp2_det(t).double()
    ref = torch.exp2(t.double())
    assert ((got - ref).abs() / ref).max().item() < 3e-7
    edge = orc.exp2_det(torch.tensor([0.0, -1.0, -126.0, float("-inf"), float("nan"), -125.0]))
    assert edge.tolist()[:4] == [1.0, 0.5, 0.0, 0.0] and edge[4].item() == 0.0
    assert edge[5].item() == 2.0 ** -125


def test_log_det_accuracy():
    v = torch.tensor(np.geomspace(1.0, 1e6, 5001), dtype=torch.float32)
    got = orc.log_det(v).double()
    ref = torch.log(v.double())
    assert (got - ref).abs().max().item() < 1e-6
    assert orc.log_det(torch.tensor([1.0])).item() == 0.0


def test_rms_norm_block_size_invariance_and_accuracy():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(8, 256, generator=g)
    r = torch.randn(8, 256, generator=g)
    w = 1.0 + 0.1 * torch.randn(256, generator=g)
    y, nr = orc.rms_norm(x, w, 1e-6, r)
    s = x + r
    ref = s * w / torch.sqrt((s * s).mean(-1, keepdim=True) + 1e-6)
    assert torch.allclose(y, ref, atol=5e-4, rtol=5e-4)
    assert torch.equal(nr, s)
    # permuting the row (with its weights) permutes the output: the sum is order-free
    perm = torch.randperm(256, generator=g)
    y2, _ = orc.rms_norm(x[:, perm], w[perm], 1e-6, r[:, perm])
    assert torch.equal(y2, y[:, perm])


def test_log_softmax_matches_float():
    g = torch.Generator().manual_seed(1)
    x = 2.0 * torch.randn(4, 1000, generator=g)
    got = orc.log_softmax(x)
    ref = torch.log_softmax(x.double(), -1)
    assert (got.double() - ref).abs().max().item() < 2e-3
    perm = torch.randperm(1000, generator=g)
    assert torch.equal(orc.log_softmax(x[:, perm]), got[:, perm])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_gemm_oracle_tile_permutation_and_tp_sharding(dtype):
    g = torch.Generator().manual_seed(2)
    kt = orc.GEMM_BLOCK_K[dtype]
    a = torch.randn(5, 4 * kt, generator=g).to(dtype)
    b = (0.1 * torch.randn(4 * kt, 7, generator=g)).to(dtype)
    bias = torch.randn(7, generator=g).to(dtype)
    c = orc.gemm_fxp(a, b, bias, 64, 16)
    ref = (a.float() @ b.float() + bias.float())
    assert torch.allclose(c.float(), ref, atol=5e-2, rtol=5e-2)
    tperm = torch.randperm(4, generator=g)
    idx = torch.cat([torch.arange(t * kt, (t + 1) * kt) for t in tperm])
    assert torch.equal(orc.gemm_fxp(a[:, idx], b[idx], bias, 64, 16), c)
    for tp in (1, 2, 4):
        assert torch.equal(orc.tp_row_parallel(a, b, bias, tp, 64, 16), c)
    # sequential and matmul partials differ at most in the last ulp -> <= few LSB
    ci = orc.gemm_fxp(a, b, None, 64, 16, return_int=True)
    cs = orc.gemm_fxp(a, b, None, 64, 16, sequential=True, return_int=True)
    assert (ci - cs).abs().max().item() <= 4


def test_gemm_int32_wraps_and_saturates_per_tile():
    a = torch.full((1, 128), 100.0)
    b = torch.full((128, 1), 100.0)
    # per-tile partial 64 * 1e4 saturates Q16.16/int32; two tiles wrap around
    acc = orc.gemm_fxp(a, b, None, 32, 16, k_tile=64, return_int=True)
    assert acc.item() == ((2**31 - 1) * 2 + 2**31) % 2**32 - 2**31


def test_attention_oracle_vs_float_softmax():
    g = torch.Generator().manual_seed(3)
    hq, hkv, d, page = 4, 2, 32, 16
    seq = [40, 70]
    blocks = [-(-s // page) for s in seq]
    kv = torch.randn(sum(blocks) + 1, 2, page, hkv, d, generator=g)
    bt = torch.zeros(2, max(blocks), dtype=torch.int32)
    order = torch.randperm(sum(blocks), generator=g) + 1
    o = 0
    for r, nb in enumerate(blocks):
        bt[r, :nb] = order[o:o + nb].int()
        o += nb
    # request 0: decode (1 token), request 1: prefill chunk of 5 tokens
    qsl = torch.tensor([0, 1, 6], dtype=torch.int32)
    q = torch.randn(6, hq, d, generator=g)
    out = orc.attention_fxp(q, kv, qsl, torch.tensor(seq, dtype=torch.int32), bt)
    for r, (q0, q1) in enumerate([(0, 1), (1, 6)]):
        s = seq[r]
        pos = torch.arange(s)
        k = kv[bt[r, pos // page].long(), 0, pos % page]
        v = kv[bt[r, pos // page].long(), 1, pos % page]
        for h in range(hq):
            sc = (q[q0:q1, h] @ k[:, h // 2].T) / math.sqrt(d)
            rows = s - (q1 - q0) + torch.arange(q1 - q0)
            sc = sc.masked_fill(pos[None, :] > rows[:, None], float("-inf"))
            ref = torch.softmax(sc, -1) @ v[:, h // 2]
            assert torch.allclose(out[q0:q1, h], ref, atol=2e-3, rtol=2e-3)
