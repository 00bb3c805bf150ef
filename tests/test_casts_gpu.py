"""GPU parity of the cast kernels: bit-exact against the CPU oracle and the
reference's known answers (mirrors fxpr_vllm/_tests/test_fixed_point_cast.py and
test_sum.py of the reference)."""
from __future__ import annotations

import json
from pathlib import Path

import pytest
import torch

from oracle import fxp_oracle as orc

pytestmark = pytest.mark.gpu
GOLD = json.loads((Path(__file__).parent / "golden" / "cast_known_answers.json").read_text())


def _h():
    import fxp_helpers
    return fxp_helpers


@pytest.mark.parametrize("case", GOLD["float_to_fixed"])
def test_known_values(case):
    x = torch.tensor(case["x"], device="cuda", dtype=torch.float32)
    got = _h().float_to_fixed(x, torch.int32, case["frac_bits"])
    assert got.cpu().tolist() == case["q"]


def test_saturation_exact_limits():
    x = torch.tensor([1e30, -1e30, 0.0, float("nan")], device="cuda")
    assert _h().float_to_fixed(x, torch.int32).cpu().tolist() == [2**31 - 1, -(2**31), 0, 0]
    assert _h().float_to_fixed(x, torch.int16, 8).cpu().tolist() == [32767, -32768, 0, 0]
    assert _h().float_to_fixed(x, torch.int64, 32).cpu().tolist() == [2**63 - 1, -(2**63), 0, -(2**63)]


@pytest.mark.parametrize("case", GOLD["float_roundtrip_exact"])
def test_roundtrip_exact(case):
    h = _h()
    x = torch.tensor(case["x"], device="cuda", dtype=torch.float32)
    it = {32: torch.int32, 64: torch.int64}[case["int_bits"]]
    back = h.fixed_to_float(h.float_to_fixed(x, it, case["frac_bits"]), torch.float32, case["frac_bits"])
    assert torch.equal(back, x)


@pytest.mark.parametrize("in_dtype", [torch.float16, torch.float32, torch.float64])
@pytest.mark.parametrize("int_dtype", [torch.int16, torch.int32, torch.int64])
@pytest.mark.parametrize("frac", [8, 16, 32])
@pytest.mark.parametrize("n", [1, 7, 1000, 8 * 256 * 3 + 5, 1 << 20])
def test_float_to_fixed_matches_oracle(in_dtype, int_dtype, frac, n):
    g = torch.Generator().manual_seed(n + frac)
    x = (torch.randn(n, generator=g, dtype=torch.float64) * 40.0).to(in_dtype)
    x[:: max(1, n // 13)] *= 1e4  # some values saturate
    got = _h().float_to_fixed(x.cuda(), int_dtype, frac).cpu()
    exp = orc.float_to_fixed(x, _h().INT_BITS[int_dtype], frac)
    assert torch.equal(got, exp)


@pytest.mark.parametrize("int_dtype", [torch.int16, torch.int32, torch.int64])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32, torch.float64])
@pytest.mark.parametrize("n", [3, 4099, 1 << 20])
def test_fixed_to_float_matches_oracle(int_dtype, out_dtype, n):
    g = torch.Generator().manual_seed(n)
    info = torch.iinfo(int_dtype)
    q = torch.randint(max(info.min, -(2**40)), min(info.max, 2**40), (n,), generator=g,
                      dtype=torch.int64).to(int_dtype)
    got = _h().fixed_to_float(q.cuda(), out_dtype, 16).cpu()
    exp = orc.fixed_to_float(q, _h().FLOAT_BITS[out_dtype], 16)
    assert torch.equal(got.view(torch.uint8), exp.view(torch.uint8))


def test_unaligned_view_and_empty():
    h = _h()
    base = torch.randn(1025, device="cuda")
    x = base[1:]  # 4-byte aligned only
    assert torch.equal(h.float_to_fixed(x, torch.int64).cpu(), orc.float_to_fixed(x.cpu(), 64, 16))
    e = torch.empty((0, 4), device="cuda")
    out = h.float_to_fixed(e, torch.int32)
    assert out.shape == (0, 4) and out.dtype == torch.int32


def test_errors_match_reference_contract():
    x = torch.randn(4, device="cuda")
    with pytest.raises(ValueError):
        torch.ops.fxpr.float_to_fixed(x, 24, 16)
    with pytest.raises(ValueError):
        torch.ops.fxpr.float_to_fixed(x, 32, 12)
    with pytest.raises(TypeError):
        torch.ops.fxpr.float_to_fixed(x.to(torch.bfloat16), 32, 16)
    with pytest.raises(ValueError):
        torch.ops.fxpr.fixed_to_float(x.to(torch.int32), 8, 16)
    with pytest.raises(TypeError):
        torch.ops.fxpr.fixed_to_float(x, 32, 16)
    with pytest.raises(NotImplementedError):
        torch.ops.fxpr.float_to_fixed(x.cpu(), 32, 16)


@pytest.mark.parametrize("case", GOLD["sum_saturates"])
def test_sum_saturates(case):
    x = torch.tensor(case["x"], device="cuda")
    s = _h().float_to_fixed(x, torch.int32).to(torch.int64).sum()
    assert int(s.clamp(-(2**31), 2**31 - 1)) == case["clamped_sum"]


def test_full_size_roundtrip_property():
    # config-0 sized tensor: decode(encode(x)) is within half a step and encode is idempotent
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((2048, 4096), device="cuda", generator=g)
    h = _h()
    q = h.float_to_fixed(x, torch.int64)
    back = h.fixed_to_float(q, torch.float32)
    assert (back - x).abs().max().item() <= 2.0 ** -17
    assert torch.equal(h.float_to_fixed(back, torch.int64), q)
