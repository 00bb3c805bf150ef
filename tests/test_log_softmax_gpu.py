"""GPU parity of the integer-sum log-softmax: bit-exact against the CPU oracle
for every cluster size / slice layout the launcher can pick."""
from __future__ import annotations

import pytest
import torch

import fxpr_vllm  # noqa: F401
from oracle import fxp_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(3, 1), (2, 5), (4, 1000), (3, 16384), (2, 16385), (2, 40001),
                                   (2, 128256), (1, 500000)])
def test_matches_oracle_bit_exact(dtype, shape):
    g = torch.Generator().manual_seed(shape[1])
    x = (2.0 * torch.randn(shape, generator=g)).to(dtype)
    got = torch.ops.fxpr.log_softmax_fxp(x.cuda(), 16).cpu()
    exp = orc.log_softmax(x, 16)
    assert got.dtype == torch.float32
    assert torch.equal(got.view(torch.int32), exp.view(torch.int32))


@pytest.mark.parametrize("frac", [8, 32])
def test_other_q_formats(frac):
    g = torch.Generator().manual_seed(frac)
    x = 3.0 * torch.randn((3, 3000), generator=g)
    got = torch.ops.fxpr.log_softmax_fxp(x.cuda(), frac).cpu()
    assert torch.equal(got.view(torch.int32), orc.log_softmax(x, frac).view(torch.int32))


def test_config3b_full_size_properties():
    g = torch.Generator(device="cuda").manual_seed(0)
    x = 2.0 * torch.randn((256, 128256), device="cuda", generator=g)
    y = torch.ops.fxpr.log_softmax_fxp(x, 16)
    assert torch.equal(y, torch.ops.fxpr.log_softmax_fxp(x, 16))
    ref = torch.log_softmax(x, dim=-1)
    # Q16.16 rounds each of the 128k terms to 2^-17: the sum, hence the log, moves by ~1e-2
    assert (y - ref).abs().max().item() < 2e-2
    # order-free: permuting the vocabulary permutes the output bit for bit
    perm = torch.randperm(128256, device="cuda", generator=g)
    assert torch.equal(torch.ops.fxpr.log_softmax_fxp(x[:, perm].contiguous(), 16), y[:, perm])
    # a few rows against the CPU oracle
    rows = [0, 100, 255]
    exp = orc.log_softmax(x[rows].cpu(), 16)
    assert torch.equal(y[rows].cpu().view(torch.int32), exp.view(torch.int32))


def test_leading_dims_and_errors():
    x = torch.randn(2, 3, 50, device="cuda")
    y = torch.ops.fxpr.log_softmax_fxp(x, 16)
    assert y.shape == x.shape
    assert torch.equal(y.cpu().view(torch.int32), orc.log_softmax(x.cpu(), 16).view(torch.int32))
    with pytest.raises(ValueError):
        torch.ops.fxpr.log_softmax_fxp(x, 12)
    with pytest.raises(TypeError):
        torch.ops.fxpr.log_softmax_fxp(x.double(), 16)
