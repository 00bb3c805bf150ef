"""GPU parity of the fixed-point GEMM.

* CUDA-core route: bit-exact against the CPU oracle (same ascending-k order).
* tensor-core route: integer stage bit-exact given the kernel's own fp32
  partials; end to end within a few Q-format LSB of the oracle (different
  in-tile summation order); bitwise invariant to split-K, batch size, K-tile
  order and repeats.
* the reference's own tests (fxpr_vllm/_tests/test_gemm.py) re-stated.
"""
from __future__ import annotations

import pytest
import torch

import fxpr_vllm  # noqa: F401
from fxpr_vllm import _lib as L
from oracle import fxp_oracle as orc

pytestmark = pytest.mark.gpu

_TOL = {torch.float32: (5e-4, 5e-4), torch.float16: (1e-2, 1e-2), torch.bfloat16: (5e-2, 5e-2)}
_DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _gemm(a, b, bias=None, int_bits=32, frac_bits=16):
    return torch.ops.fxpr.gemm_fxp(a, b, bias, int_bits, frac_bits)


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


# ---------------- CUDA-core route: bit-exact vs oracle -----------------------------

@pytest.mark.parametrize("dtype", _DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 1, 32), (3, 7, 16), (4, 4, 33), (130, 130, 33), (65, 200, 300)])
@pytest.mark.parametrize("int_bits", [16, 32, 64])
def test_portable_bit_exact(dtype, M, N, K, int_bits):
    a = _rand((M, K), dtype, 1, 0.5)
    b = _rand((K, N), dtype, 2, 0.5)
    bias = _rand((N,), dtype, 3)
    with L.overrides(gemm_portable=True):
        got = _gemm(a.cuda(), b.cuda(), bias.cuda(), int_bits, 16).cpu()
        got_int = torch.ops.fxpr.gemm_fxp_int(a.cuda(), b.cuda(), int_bits, 16).cpu()
    exp_int = orc.gemm_fxp(a, b, None, int_bits, 16, sequential=True, return_int=True)
    assert torch.equal(got_int.to(torch.int64), exp_int)
    exp = orc.gemm_epilogue(exp_int, bias, dtype, 16)
    assert torch.equal(got.view(torch.uint8), exp.view(torch.uint8))


def test_portable_strided_operands():
    a = _rand((40, 96), torch.float32, 4)
    w = _rand((24, 96), torch.float32, 5)  # (N, K) weight viewed as (K, N)
    with L.overrides(gemm_portable=True):
        got = _gemm(a.cuda()[::2], w.cuda().t(), None, 64, 16).cpu()
    exp = orc.gemm_fxp(a[::2], w.t(), None, 64, 16, sequential=True)
    assert torch.equal(got, exp)


# ---------------- default route: tolerance + invariance (all dtypes) ----------------

@pytest.mark.parametrize("dtype", _DTYPES)
@pytest.mark.parametrize("M,N,K", [(8, 16, 32), (4, 4, 64), (130, 130, 33), (256, 256, 256),
                                   (100, 384, 512), (300, 264, 1096)])
@pytest.mark.parametrize("use_bias", [False, True])
def test_matches_float_matmul(dtype, M, N, K, use_bias):
    a = _rand((M, K), dtype, 11, 0.5).cuda()
    b = _rand((K, N), dtype, 12, 0.5).cuda()
    bias = _rand((N,), dtype, 13).cuda() if use_bias else None
    got = _gemm(a, b, bias)
    assert got.dtype == dtype and got.shape == (M, N)
    ref = a.float() @ b.float()
    if use_bias:
        ref = ref + bias.float()
    atol, rtol = _TOL[dtype]
    assert torch.allclose(got.float(), ref.to(dtype).float(), atol=atol * max(1.0, K / 64) ** 0.5,
                          rtol=rtol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K,kt", [(128, 256, 512, 64), (200, 320, 1024, 128), (64, 4096, 1024, 64)])
def test_int_accumulators_close_to_oracle(dtype, M, N, K, kt):
    a = _rand((M, K), dtype, 21).cuda()
    b = _rand((K, N), dtype, 22, 0.05).cuda()
    with L.overrides(gemm_k_tile=kt, gemm_split_k=1):
        got = torch.ops.fxpr.gemm_fxp_int(a, b, 64, 16).cpu()
    exp = orc.gemm_fxp(a.cpu(), b.cpu(), None, 64, 16, k_tile=kt, return_int=True)
    # each K-tile's partial can differ in its last fp32 ulp -> at most one LSB per tile
    assert (got - exp).abs().max().item() <= K // kt
    assert (got - exp).abs().float().mean().item() < 0.25


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("int_bits", [32, 64])
def test_integer_stage_exact_given_kernel_partials(dtype, int_bits):
    M, N, K, kt = 150, 264, 640, 64
    a = _rand((M, K), dtype, 31, 2.0).cuda()
    b = _rand((K, N), dtype, 32, 2.0).cuda()
    a[0, :] = 3000.0  # rows that saturate a Q16.16/int32 tile and wrap the sum
    b[:, 0] = 3000.0
    with L.overrides(gemm_k_tile=kt, gemm_split_k=1, gemm_partials=True) as o:
        got = torch.ops.fxpr.gemm_fxp_int(a, b, int_bits, 16).cpu()
        partials = o.last_partials.cpu()
    exp = orc.gemm_int_from_partials(partials, int_bits, 16)
    assert torch.equal(got.to(torch.int64), exp)


@pytest.mark.parametrize("dtype", _DTYPES)
def test_deterministic_across_runs(dtype):
    a = _rand((200, 512), dtype, 41).cuda()
    b = _rand((512, 136), dtype, 42).cuda()
    first = _gemm(a, b)
    for _ in range(4):
        assert torch.equal(first, _gemm(a, b))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(64, 512, 2048), (300, 264, 1096), (1, 128, 4096)])
@pytest.mark.parametrize("kt", [64, 128])
def test_split_k_invariance(dtype, M, N, K, kt):
    a = _rand((M, K), dtype, 51).cuda()
    b = _rand((K, N), dtype, 52, 0.05).cuda()
    bias = _rand((N,), dtype, 53).cuda()
    outs = []
    for split in (1, 2, 4, 8, 16):
        with L.overrides(gemm_k_tile=kt, gemm_split_k=split):
            outs.append((_gemm(a, b, bias, 64, 16), torch.ops.fxpr.gemm_fxp_int(a, b, 64, 16)))
    for c, ci in outs[1:]:
        assert torch.equal(c, outs[0][0]) and torch.equal(ci, outs[0][1])
    # scratch is left clean: a second sweep gives the same bits
    with L.overrides(gemm_k_tile=kt, gemm_split_k=4):
        assert torch.equal(_gemm(a, b, bias, 64, 16), outs[0][0])


@pytest.mark.parametrize("dtype", _DTYPES)
def test_ktile_permutation_invariance(dtype):
    kt = L.BLOCK_K_BY_DTYPE[dtype]
    M, K, N = 4, kt * 4, 8
    a = _rand((M, K), dtype, 61).cuda()
    b = _rand((K, N), dtype, 62).cuda()
    tperm = torch.randperm(4)
    perm = torch.cat([torch.arange(t * kt, (t + 1) * kt) for t in tperm]).cuda()
    assert torch.equal(_gemm(a, b), _gemm(a[:, perm].contiguous(), b[perm].contiguous()))


@pytest.mark.parametrize("dtype", _DTYPES)
@pytest.mark.parametrize("K,N", [(64, 16), (512, 264)])
def test_batch_size_invariance(dtype, K, N):
    a_full = _rand((300, K), dtype, 71).cuda()
    b = _rand((K, N), dtype, 72).cuda()
    rows = [0, 3, 17, 64, 127, 299]
    refs = {m: _gemm(a_full[m:m + 1], b)[0] for m in rows}
    for batch in (1, 4, 16, 128, 300):
        out = _gemm(a_full[:batch], b)
        for m in rows:
            if m < batch:
                assert torch.equal(out[m], refs[m]), f"row {m} differs at batch={batch}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_tensor_core_route_agrees_with_cuda_core_route(dtype):
    a = _rand((96, 512), dtype, 81).cuda()
    b = _rand((512, 128), dtype, 82, 0.1).cuda()
    tc = torch.ops.fxpr.gemm_fxp_int(a, b, 64, 16)
    with L.overrides(gemm_portable=True):
        cc = torch.ops.fxpr.gemm_fxp_int(a, b, 64, 16)
    assert (tc - cc).abs().max().item() <= 512 // L.BLOCK_K_BY_DTYPE[dtype]


def test_identity_zero_and_empty():
    a = _rand((4, 16), torch.float32, 91).cuda()
    assert torch.allclose(_gemm(a, torch.eye(16, device="cuda")), a, atol=1e-4)
    z = _gemm(torch.ones((4, 16), device="cuda"), torch.zeros((16, 4), device="cuda"))
    assert torch.equal(z, torch.zeros((4, 4), device="cuda"))
    e = _gemm(torch.empty((0, 16), device="cuda"), torch.zeros((16, 4), device="cuda"))
    assert e.shape == (0, 4)
    with pytest.raises(ValueError):
        _gemm(a, torch.eye(16, device="cuda"), None, 24, 16)


def test_epilogue_from_int_matches_oracle():
    g = torch.Generator().manual_seed(5)
    ci = torch.randint(-(2**40), 2**40, (37, 53), generator=g, dtype=torch.int64)
    bias = torch.randn(53, generator=g).to(torch.bfloat16)
    got = torch.ops.fxpr.gemm_fxp_epilogue(ci.cuda(), bias.cuda(), torch.bfloat16, 16).cpu()
    exp = orc.gemm_epilogue(ci, bias, torch.bfloat16, 16)
    assert torch.equal(got.view(torch.uint8), exp.view(torch.uint8))


def test_tp_sharding_single_gpu_equals_unsharded():
    # row-parallel layer: K sharded over "ranks", integer accumulators summed
    a = _rand((64, 4096), torch.bfloat16, 95).cuda()
    b = _rand((4096, 512), torch.bfloat16, 96, 0.02).cuda()
    full = torch.ops.fxpr.gemm_fxp_int(a, b, 64, 16)
    for tp in (2, 4, 8):
        ks = 4096 // tp
        acc = torch.zeros_like(full)
        for r in range(tp):
            acc += torch.ops.fxpr.gemm_fxp_int(a[:, r * ks:(r + 1) * ks], b[r * ks:(r + 1) * ks], 64, 16)
        assert torch.equal(acc, full)
    out = torch.ops.fxpr.gemm_fxp_epilogue(full, None, torch.bfloat16, 16)
    assert torch.equal(out, _gemm(a, b, None, 64, 16))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("int_bits", [32, 64])
@pytest.mark.parametrize("kt,split", [(64, 1), (128, 1), (64, 3), (128, 2)])
@pytest.mark.parametrize("tile", ["n128", "n256", "pair128", "pair256"])
def test_fast_epilogue_equals_plain_conversion_with_outliers(dtype, int_bits, kt, split, tile):
    """The magic-number epilogue with its exact fix-up gives the same integers as the
    tensor-core kernel that converts every partial with cvt.rni (saturating), including
    rows whose partials leave the fast range, saturate int32 or overflow the 32-bit sum."""
    from fxpr_vllm import _native as nat

    M, N, K = 300, 520, 1096
    a = _rand((M, K), dtype, 101).cuda()
    b = _rand((K, N), dtype, 102, 0.05).cuda()
    a[3, :] = 900.0
    a[M - 1, 5::7] = -3000.0
    a[M // 2, :64] = 6.0e4
    a[7, 100] = float("inf") if int_bits == 32 else 5.0e4
    # every tile shape, whatever the default: 128 x 128, 128 x 256, and the two-SM kernel's
    # 256 x 128 / 256 x 256 pair tiles
    shape_flag = {"n128": nat.GEMM_TILE_N128, "n256": nat.GEMM_TILE_N256,
                  "pair128": nat.GEMM_PAIR | nat.GEMM_TILE_N128, "pair256": nat.GEMM_PAIR}[tile]
    with L.overrides(gemm_k_tile=kt, gemm_split_k=split, gemm_flags=shape_flag):
        fast_i = torch.ops.fxpr.gemm_fxp_int(a, b, int_bits, 16)
        fast_c = _gemm(a, b, None, int_bits, 16)
    with L.overrides(gemm_k_tile=kt, gemm_split_k=1, gemm_flags=nat.GEMM_FORCE_EXACT_TC):
        exact_i = torch.ops.fxpr.gemm_fxp_int(a, b, int_bits, 16)
        exact_c = _gemm(a, b, None, int_bits, 16)
    assert torch.equal(fast_i, exact_i)
    assert torch.equal(fast_c.view(torch.int16), exact_c.view(torch.int16))
    L.check_device_status()


@pytest.mark.parametrize("int_bits,frac", [(16, 8), (64, 32), (32, 8)])
def test_tensor_core_route_other_q_formats(int_bits, frac):
    a = _rand((130, 512), torch.bfloat16, 111, 0.3).cuda()
    b = _rand((512, 264), torch.bfloat16, 112, 0.1).cuda()
    got = torch.ops.fxpr.gemm_fxp_int(a, b, int_bits, frac).cpu().to(torch.int64)
    exp = orc.gemm_fxp(a.cpu(), b.cpu(), None, int_bits, frac, return_int=True)
    tol = 4 if frac <= 16 else 4 * 2 ** (frac - 16)
    assert (got - exp).abs().max().item() <= tol


def test_b_given_as_transposed_weight_view():
    # weight kept (N, K) and passed as .t(): the K-major operand path, no transpose copy
    a = _rand((200, 1024), torch.bfloat16, 121).cuda()
    w = _rand((384, 1024), torch.bfloat16, 122, 0.05).cuda()
    v1 = torch.ops.fxpr.gemm_fxp_int(a, w.t(), 64, 16)
    v2 = torch.ops.fxpr.gemm_fxp_int(a, w.t().contiguous(), 64, 16)
    assert torch.equal(v1, v2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [1, 16, 33, 64])
@pytest.mark.parametrize("kt,split", [(64, 1), (128, 1), (64, 3), (128, 4), (64, 8), (128, 2), (64, 2)])
@pytest.mark.parametrize("int_bits", [32, 64])
def test_decode_shape_kernel_equals_wide_tile_kernel(dtype, M, kt, split, int_bits):
    """M <= 64 goes to the kernel that puts the weights on the 128-row side of the MMA.  Its
    integers and outputs must be those of the 128-row-tile kernel (and hence do not depend on
    how many rows share the launch), for both weight layouts, with bias, a ragged N and K,
    split-K and partials outside the fast conversion's range."""
    from fxpr_vllm import _native as nat

    N, K = 520, 1096
    a = _rand((M, K), dtype, 201).cuda()
    b = _rand((K, N), dtype, 202, 0.05).cuda()
    bias = _rand((N,), dtype, 203).cuda()
    a[0, 5::7] = -3000.0
    a[M - 1, :64] = 6.0e4
    bt_view = b.t().contiguous().t()               # (K, N) view of an (N, K) row-major matrix
    for bb in (b, bt_view):
        with L.overrides(gemm_k_tile=kt, gemm_split_k=split):
            sk_i = torch.ops.fxpr.gemm_fxp_int(a, bb, int_bits, 16)
            sk_c = _gemm(a, bb, bias, int_bits, 16)
        with L.overrides(gemm_k_tile=kt, gemm_split_k=1, gemm_flags=nat.GEMM_NO_SKINNY):
            wide_i = torch.ops.fxpr.gemm_fxp_int(a, bb, int_bits, 16)
            wide_c = _gemm(a, bb, bias, int_bits, 16)
        assert torch.equal(sk_i, wide_i)
        assert torch.equal(sk_c.view(torch.int16), wide_c.view(torch.int16))
        if split > 1:      # 2/4/8 splits merge inside a cluster by default; the scratch-plane merge must agree
            with L.overrides(gemm_k_tile=kt, gemm_split_k=split, gemm_flags=nat.GEMM_NO_CLUSTER):
                pl_i = torch.ops.fxpr.gemm_fxp_int(a, bb, int_bits, 16)
            assert torch.equal(pl_i, wide_i)
    L.check_device_status()


def test_decode_row_bits_do_not_depend_on_the_batch():
    """Row r of a 64-row launch (decode-shape kernel) equals row r of a 300-row launch."""
    a = _rand((300, 1024), torch.bfloat16, 211).cuda()
    b = _rand((1024, 384), torch.bfloat16, 212, 0.05).cuda()
    big = _gemm(a, b, None, 64, 16)
    small = _gemm(a[100:164].contiguous(), b, None, 64, 16)
    assert torch.equal(small.view(torch.int16), big[100:164].view(torch.int16))


def test_routes_agree_on_random_shapes():
    """Seeded sweep over ragged shapes: whichever kernel the dispatcher picks (decode-shape,
    128x128 or 128x256 tiles, cluster or plane split-K) must give the integers of the
    tensor-core kernel with plain cvt.rni conversion, for both weight layouts."""
    from fxpr_vllm import _native as nat

    g = torch.Generator().manual_seed(2024)
    for case in range(40):
        M = int(torch.randint(1, 400, (1,), generator=g))
        if case % 3 == 0:
            M = int(torch.randint(1, 65, (1,), generator=g))
        N = 8 * int(torch.randint(8, 130, (1,), generator=g))
        K = 8 * int(torch.randint(8, 300, (1,), generator=g))
        kt = (64, 128)[case % 2]
        split = (1, 2, 3, 4, 8)[case % 5]
        int_bits = (64, 32)[(case // 2) % 2]
        dtype = (torch.bfloat16, torch.float16)[(case // 4) % 2]
        a = _rand((M, K), dtype, 1000 + case).cuda()
        b = _rand((K, N), dtype, 2000 + case, 0.05).cuda()
        if case % 7 == 0:
            a[M // 2, : min(64, K)] = 3.0e4
        bb = b if case % 2 else b.t().contiguous().t()
        with L.overrides(gemm_k_tile=kt, gemm_split_k=split):
            got = torch.ops.fxpr.gemm_fxp_int(a, bb, int_bits, 16)
        with L.overrides(gemm_k_tile=kt, gemm_split_k=1, gemm_flags=nat.GEMM_FORCE_EXACT_TC):
            exp = torch.ops.fxpr.gemm_fxp_int(a, bb, int_bits, 16)
        assert torch.equal(got, exp), (case, M, N, K, kt, split, int_bits, dtype)
    L.check_device_status()


def test_two_sm_kernel_agrees_on_random_shapes():
    """The cta_group::2 kernel (CTA pairs, 256-row tiles) gives the integers of the plain-conversion
    tensor-core kernel on ragged shapes, with and without split-K, for both weight layouts."""
    from fxpr_vllm import _native as nat

    g = torch.Generator().manual_seed(77)
    for case in range(24):
        M = int(torch.randint(129, 900, (1,), generator=g))
        N = 8 * int(torch.randint(16, 130, (1,), generator=g))
        K = 8 * int(torch.randint(8, 300, (1,), generator=g))
        kt = (64, 128)[case % 2]
        split = (1, 2, 3, 5)[case % 4]
        int_bits = (64, 32)[(case // 2) % 2]
        dtype = (torch.bfloat16, torch.float16)[(case // 4) % 2]
        flag = nat.GEMM_PAIR | (nat.GEMM_TILE_N128 if case % 3 == 0 else 0)
        a = _rand((M, K), dtype, 3000 + case).cuda()
        b = _rand((K, N), dtype, 4000 + case, 0.05).cuda()
        if case % 5 == 0:
            a[M // 2, : min(64, K)] = 3.0e4
        bb = b if case % 2 else b.t().contiguous().t()
        bias = _rand((N,), dtype, 5000 + case).cuda() if case % 2 else None
        with L.overrides(gemm_k_tile=kt, gemm_split_k=split, gemm_flags=flag):
            got = torch.ops.fxpr.gemm_fxp_int(a, bb, int_bits, 16)
            got_c = _gemm(a, bb, bias, int_bits, 16)
        with L.overrides(gemm_k_tile=kt, gemm_split_k=1, gemm_flags=nat.GEMM_FORCE_EXACT_TC):
            exp = torch.ops.fxpr.gemm_fxp_int(a, bb, int_bits, 16)
            exp_c = _gemm(a, bb, bias, int_bits, 16)
        assert torch.equal(got, exp), (case, M, N, K, kt, split, int_bits, dtype)
        assert torch.equal(got_c.view(torch.int16), exp_c.view(torch.int16)), case
    L.check_device_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,f,K", [(64, 1792, 1024), (33, 200, 512), (1, 128, 256), (64, 4096, 2048)])
@pytest.mark.parametrize("split", [0, 1, 2, 3, 4])
def test_silu_mul_epilogue_equals_gemm_then_silu_mul(dtype, M, f, K, split):
    """The decode-shape GEMM with (gate, up) column pairs and SiLU*mul in its epilogue gives the
    bits of the plain GEMM on [gate | up] followed by the SiLU*mul kernel, for every split
    route (one CTA per tile, cluster merge, partial planes), and so does the two-kernel form on
    the paired layout that larger batches take."""
    from fxpr_vllm import _lib as L

    g = torch.Generator().manual_seed(M * 7 + f)
    a = torch.randn(M, K, generator=g).to(dtype).cuda()
    wg = (0.05 * torch.randn(K, f, generator=g)).to(dtype).cuda()
    wu = (0.05 * torch.randn(K, f, generator=g)).to(dtype).cuda()
    kw = {} if split == 0 else {"gemm_split_k": split}
    with L.overrides(gemm_k_tile=128, **kw):
        want = L.silu_mul(torch.ops.fxpr.gemm_fxp(a, torch.cat([wg, wu], dim=1).contiguous(), None, 64, 16))
        pairs = L.interleave_gate_up(wg, wu)
        got = L.gemm_silu_mul(a, pairs, 64, 16)
        two = L.silu_mul_pairs(torch.ops.fxpr.gemm_fxp(a, pairs, None, 64, 16))
    assert got.shape == (M, f)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert torch.equal(two.view(torch.int16), want.view(torch.int16))


def test_silu_mul_epilogue_falls_back_for_large_batches():
    from fxpr_vllm import _lib as L

    g = torch.Generator().manual_seed(3)
    a = torch.randn(200, 512, generator=g).to(torch.bfloat16).cuda()
    wg = (0.05 * torch.randn(512, 384, generator=g)).to(torch.bfloat16).cuda()
    wu = (0.05 * torch.randn(512, 384, generator=g)).to(torch.bfloat16).cuda()
    want = L.silu_mul(torch.ops.fxpr.gemm_fxp(a, torch.cat([wg, wu], dim=1).contiguous(), None, 64, 16))
    got = L.gemm_silu_mul(a, L.interleave_gate_up(wg, wu), 64, 16)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(64, 16032, 512), (33, 1000, 256), (1, 128, 128), (64, 4096, 1024)])
def test_gemm_argmax_keys_equal_argmax_of_the_logits(dtype, M, N, K):
    """The lm_head GEMM that also leaves per-row arg-max keys: same logits as ``gemm_fxp``, the
    winning column equals ``torch.argmax`` of them (first maximal column: the weights hold
    duplicated columns, so every row has ties), and the keys of two column shards combine to the
    key of the whole row."""
    from fxpr_vllm import _lib as L

    g = torch.Generator().manual_seed(N + M)
    a = torch.randn(M, K, generator=g).to(dtype).cuda()
    b = (0.05 * torch.randn(K, N, generator=g)).to(dtype)
    b[:, N // 3] = b[:, N // 2]                      # exact ties between far-apart columns
    b[:, N - 1] = b[:, 0]
    b = b.cuda()
    want = torch.ops.fxpr.gemm_fxp(a, b, None, 64, 16)
    logits, keys = L.gemm_fxp_argmax(a, b, None, 64, 16)
    assert torch.equal(logits.view(torch.int16), want.view(torch.int16))
    assert torch.equal(L.argmax_from_keys(keys), want.argmax(dim=-1))
    assert torch.equal(keys, L.argmax_keys_of(want))
    half = (N // 2 + 127) // 128 * 128 if N > 256 else N // 2
    k0 = L.gemm_fxp_argmax(a, b[:, :half].contiguous(), None, 64, 16, n_offset=0)[1]
    k1 = L.gemm_fxp_argmax(a, b[:, half:].contiguous(), None, 64, 16, n_offset=half)[1]
    assert torch.equal(L.combine_argmax_keys([k0, k1]), keys)
    big = torch.randn(100, K, generator=g).to(dtype).cuda()      # more than 64 rows: two-kernel form
    lg2, k2 = L.gemm_fxp_argmax(big, b, None, 64, 16)
    assert torch.equal(L.argmax_from_keys(k2), lg2.argmax(dim=-1))


@pytest.mark.parametrize("split", [0, 1, 4])
def test_static_weights_promise_changes_no_bit(split):
    """With FXPR_GEMM_WEIGHTS_STATIC the decode-shape kernel only moves its first weight requests
    in front of the dependency wait; the outputs are the same, also back to back in one stream
    with a kernel that writes the activations just before."""
    from fxpr_vllm import _lib as L

    g = torch.Generator().manual_seed(11)
    w = (0.05 * torch.randn(2048, 1536, generator=g)).to(torch.bfloat16).cuda()
    x0 = torch.randn(48, 2048, generator=g).cuda()
    torch.cuda.synchronize()                                # the weights are complete, as the flag promises
    kw = {} if split == 0 else {"gemm_split_k": split}
    with L.overrides(gemm_k_tile=128, **kw):
        wants = {sc: torch.ops.fxpr.gemm_fxp((x0 * sc).to(torch.bfloat16), w, None, 64, 16) for sc in (1.0, 0.5, 2.0)}
        with L.static_weights():
            for sc in (1.0, 0.5, 2.0):
                x = (x0 * sc).to(torch.bfloat16)            # written by the kernel right before the GEMM
                assert torch.equal(torch.ops.fxpr.gemm_fxp(x, w, None, 64, 16), wants[sc])
        assert torch.equal(torch.ops.fxpr.gemm_fxp(x0.to(torch.bfloat16), w, None, 64, 16), wants[1.0])
