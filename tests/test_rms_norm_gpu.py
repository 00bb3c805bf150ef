"""GPU parity of RMSNorm(+residual): bit-exact against the CPU oracle, plus the
reference's own tolerance / in-place / order-freedom tests
(fxpr_vllm/_tests/test_rms_norm.py)."""
from __future__ import annotations

import pytest
import torch

import fxpr_vllm  # noqa: F401
from oracle import fxp_oracle as orc

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.contiguous().view(torch.uint8)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 7), (3, 16), (4, 31), (5, 4096), (3, 8192), (2, 20000)])
@pytest.mark.parametrize("residual", [False, True])
def test_matches_oracle_bit_exact(dtype, shape, residual):
    g = torch.Generator().manual_seed(shape[1])
    x = torch.randn(shape, generator=g).to(dtype)
    r = torch.randn(shape, generator=g).to(dtype) if residual else None
    w = (1.0 + 0.1 * torch.randn(shape[1], generator=g)).to(dtype)
    y_exp, r_exp = orc.rms_norm(x, w, 1e-6, r)
    xc, wc = x.cuda(), w.cuda()
    if residual:
        rc = r.cuda()
        y = torch.ops.fxpr.rms_norm_fxp_residual(xc, rc, wc, 1e-6)
        assert torch.equal(_bits(rc.cpu()), _bits(r_exp))
    else:
        y = torch.ops.fxpr.rms_norm_fxp(xc, wc, 1e-6)
    assert y.dtype == dtype and y.shape == x.shape
    assert torch.equal(_bits(y.cpu()), _bits(y_exp))


def test_config0_full_size_bit_exact_and_repeatable():
    g = torch.Generator().manual_seed(0)
    x = torch.randn((2048, 4096), generator=g)
    r = torch.randn((2048, 4096), generator=g)
    w = 1.0 + 0.1 * torch.randn(4096, generator=g)
    y_exp, r_exp = orc.rms_norm(x, w, 1e-6, r)
    outs = []
    for _ in range(3):
        rc = r.cuda()
        y = torch.ops.fxpr.rms_norm_fxp_residual(x.cuda(), rc, w.cuda(), 1e-6)
        outs.append((y.cpu(), rc.cpu()))
    assert torch.equal(outs[0][0], y_exp) and torch.equal(outs[0][1], r_exp)
    for y, rr in outs[1:]:
        assert torch.equal(y, outs[0][0]) and torch.equal(rr, outs[0][1])


@pytest.mark.parametrize("shape", [(2, 7), (3, 16), (4, 31)])
def test_reference_tolerance_vs_float(shape):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.rand(shape, device="cuda", generator=g) - 0.5) * 32.0
    w = (torch.rand(shape[1], device="cuda", generator=g) - 0.5) * 4.0
    got = torch.ops.fxpr.rms_norm_fxp(x, w, 1e-6)
    ref = x * w / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6)
    assert torch.allclose(got, ref, atol=5e-4, rtol=5e-4)


def test_row_permutation_equivariance():
    x_a = torch.tensor([64.0, 1.0, 1.0, 1.0, 1.0], device="cuda")
    perm = torch.tensor([1, 2, 3, 4, 0], device="cuda")
    x = torch.stack([x_a, x_a[perm]])
    y = torch.ops.fxpr.rms_norm_fxp(x, torch.ones(5, device="cuda"), 1e-6)
    assert torch.equal(y[1], y[0][perm])


def test_nd_input_noncontiguous_residual_and_empty():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 3, 64, generator=g)
    w = torch.randn(64, generator=g)
    big = torch.randn(2, 3, 128, generator=g)
    r_view = big.cuda()[..., ::2]  # non-contiguous residual: copy-back path
    r_cpu = big[..., ::2].clone()
    y_exp, r_exp = orc.rms_norm(x, w, 1e-5, r_cpu)
    y = torch.ops.fxpr.rms_norm_fxp_residual(x.cuda(), r_view, w.cuda(), 1e-5)
    assert torch.equal(y.cpu(), y_exp) and torch.equal(r_view.cpu(), r_exp)
    e = torch.empty((0, 64), device="cuda")
    assert torch.ops.fxpr.rms_norm_fxp(e, w.cuda(), 1e-6).shape == (0, 64)


def test_errors():
    x = torch.randn(2, 8, device="cuda")
    with pytest.raises(TypeError):
        torch.ops.fxpr.rms_norm_fxp(x, torch.ones(8, device="cuda", dtype=torch.float16), 1e-6)
    with pytest.raises(TypeError):
        torch.ops.fxpr.rms_norm_fxp(x.double(), torch.ones(8, device="cuda").double(), 1e-6)
    with pytest.raises(ValueError):
        torch.ops.fxpr.rms_norm_fxp_residual(x, torch.randn(2, 4, device="cuda"),
                                             torch.ones(8, device="cuda"), 1e-6)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("int_bits", [32, 64])
@pytest.mark.parametrize("use_bias", [False, True])
def test_from_int_kernel_equals_epilogue_then_residual_norm(dtype, int_bits, use_bias):
    """``rms_norm_fxp_from_int`` (conversion of the all-reduced integer accumulators + bias +
    residual add + RMSNorm in one kernel, the step after a tensor-parallel row-parallel GEMM)
    gives the bits of ``gemm_fxp_epilogue`` followed by ``rms_norm_fxp_residual``."""
    g = torch.Generator().manual_seed(7)
    rows, hidden = 37, 4096
    idt = torch.int32 if int_bits == 32 else torch.int64
    acc = (torch.randn(rows, hidden, generator=g) * 3 * 65536).to(idt).cuda()
    res = torch.randn(rows, hidden, generator=g).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).cuda()
    bias = torch.randn(hidden, generator=g).to(dtype).cuda() if use_bias else None
    r1, r2 = res.clone(), res.clone()
    x = torch.ops.fxpr.gemm_fxp_epilogue(acc, bias, dtype, 16)
    want = torch.ops.fxpr.rms_norm_fxp_residual(x, r1, w, 1e-6)
    got = torch.ops.fxpr.rms_norm_fxp_from_int(acc, r2, w, bias, 1e-6, 16)
    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    assert torch.equal(r1.view(torch.uint8), r2.view(torch.uint8))
