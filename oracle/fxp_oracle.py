"""CPU oracle for the fixed-point reduction path -- TEST INFRASTRUCTURE ONLY.

This module restates, with torch-on-CPU / numpy arithmetic, what the reference
plugin ``fxpr_vllm`` computes on the GPU.  It exists so the CUDA kernels can be
checked bit for bit (integer stages, IEEE-only float stages) or within one
Q-format LSB (tensor-core stages).  Only the tests, the smoke entry and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark import it; the
product path never does and fails loudly without its CUDA library.

Pinning status
--------------
* ``float_to_fixed`` / ``fixed_to_float``: pinned against every known-answer
  vector in the reference's own tests (``fxpr_vllm/_tests/test_fixed_point_cast.py:7-42,
  58-67, 89-113`` and ``fxpr_vllm/_tests/test_sum.py:51-119``), stored in
  ``tests/golden/cast_known_answers.json``.
  They are also pinned, bit for bit, against outputs of the reference's own kernels
  recorded on a B200 (``tests/golden/reference_b200.pt``, made by
  ``tests/golden/make_reference_fixtures.py``).
* GEMM / attention: follow ``fxpr_vllm/_triton/gemm.py:183-204`` and
  ``fxpr_vllm/_triton/attention.py:199-301``.  The reference's tests hold no absolute
  output bits for these ops (only tolerances and self-invariance); the recorded B200
  outputs of the reference pin them to one unit in the last place of the io dtype on
  under 1 % of the elements -- the per-tile fp32 partial of the reference comes out of
  ``tl.dot`` in the tensor core's own summation order, which a sequential restatement
  cannot reproduce bit for bit.  The integer stage itself is exact.
* RMSNorm with an integer sum of squares (the reference sums in fp32,
  ``fxpr_vllm/_triton/rms_norm.py:41-50``): within one fp32 ulp of the recorded
  reference outputs, residual output bit-exact.
* Log-softmax and the tensor-parallel integer all-reduce have no reference
  implementation at all (the sampler files named in ``README.md:60,69`` do not
  exist): parity unpinned, the semantics are defined here.

Float operations used below are single IEEE-754 round-to-nearest-even
operations (no fused multiply-add), which is what the CUDA side compiles to
with ``-fmad=false`` in its "exact" kernels, so both sides agree bit for bit.
"""

from __future__ import annotations

import math

import numpy as np
import torch

RCP_LN2 = 1.4426950408889634  # fxpr_vllm/_triton/attention.py:21

_INT_DTYPE = {16: torch.int16, 32: torch.int32, 64: torch.int64}
_FLOAT_DTYPE = {16: torch.float16, 32: torch.float32, 64: torch.float64}

# K-tile (GEMM) and key-tile (attention) widths: the determinism granularity.
GEMM_BLOCK_K = {torch.float16: 128, torch.bfloat16: 128, torch.float32: 64}  # gemm.py:26-30
ATTN_BLOCK_N = {torch.float16: 64, torch.bfloat16: 64, torch.float32: 32}  # attention.py:32-36


# --------------------------------------------------------------------------
# Q-format casts
# --------------------------------------------------------------------------

def fxp_limits(int_bits: int) -> tuple[int, int]:
    """(qmin, qmax) of a signed ``int_bits`` integer; fxp.py:42-43."""
    return -(1 << (int_bits - 1)), (1 << (int_bits - 1)) - 1


def float_to_fixed(x: torch.Tensor, int_bits: int, frac_bits: int) -> torch.Tensor:
    """``int(rint_sat(fp32(x) * 2^frac))``; fxp.py:92-108, casts.py:21-37.

    The product is formed in fp32, rounded half-to-even and saturated to the
    integer range.  NaN maps to 0 on the 16/32-bit paths (PTX ``cvt`` rule) and
    to qmin on the 64-bit path (the fp32 max/min clamp drops the NaN first).
    """
    qmin, qmax = fxp_limits(int_bits)
    scaled = x.to(torch.float32) * float(1 << frac_bits)
    r = torch.round(scaled).to(torch.float64)  # half-to-even, exact in fp64
    nan = torch.isnan(r)
    # Saturate in fp64, where both limits of int16/int32 are exact; int64 limits
    # need an explicit guard because 2^63 is not an int64.
    lo, hi = float(qmin), float(qmax)
    if int_bits == 64:
        big = r >= 9.223372036854775807e18
        small = r <= -9.223372036854775808e18
        r = torch.where(big | small | nan, torch.zeros_like(r), r)
        q = r.to(torch.int64)
        q = torch.where(big, torch.full_like(q, qmax), q)
        q = torch.where(small | nan, torch.full_like(q, qmin), q)
        return q
    r = torch.where(nan, torch.zeros_like(r), r)
    r = torch.clamp(r, lo, hi)
    return r.to(torch.int64).to(_INT_DTYPE[int_bits])


def fixed_to_float(q: torch.Tensor, float_bits: int, frac_bits: int) -> torch.Tensor:
    """``T(fp32(q) * 2^-frac)``; fxp.py:111-113, casts.py:40-54."""
    y = q.to(torch.float32) * (1.0 / float(1 << frac_bits))
    return y.to(_FLOAT_DTYPE[float_bits])


def _wrap_to_bits(acc: torch.Tensor, int_bits: int) -> torch.Tensor:
    """Two's-complement wrap of an int64 sum to ``int_bits`` (plain ``+=`` in
    the reference's accumulator type, gemm.py:190)."""
    if int_bits == 64:
        return acc
    return acc.to(_INT_DTYPE[int_bits]).to(torch.int64)


# --------------------------------------------------------------------------
# Deterministic elementary functions (shared definition with the CUDA side)
# --------------------------------------------------------------------------

_EXP2_COEF = [np.float32((math.log(2.0) ** k) / math.factorial(k)) for k in range(8)]


def exp2_det(t: torch.Tensor) -> torch.Tensor:
    """2**t for fp32 ``t`` from IEEE single operations only.

    ``n = rint(t)``, ``f = t - n`` (exact), a degree-7 Horner polynomial in ``f``
    with separate multiply and add, then an exact scaling by 2**n.  Arguments
    below -125 (and NaN) give 0; arguments above 127 give +inf.
    """
    a = t.detach().to(torch.float32).numpy().astype(np.float32)
    out = np.zeros_like(a)
    ok = a >= np.float32(-125.0)
    big = a > np.float32(127.0)
    ac = np.where(ok & ~big, a, np.float32(0.0)).astype(np.float32)
    n = np.rint(ac).astype(np.float32)
    f = (ac - n).astype(np.float32)
    p = np.full_like(f, _EXP2_COEF[7])
    for k in range(6, -1, -1):
        p = (p * f).astype(np.float32)
        p = (p + _EXP2_COEF[k]).astype(np.float32)
    two_n = ((n.astype(np.int32) + 127) << 23).astype(np.int32).view(np.float32)
    res = (p * two_n).astype(np.float32)
    out = np.where(ok, res, np.float32(0.0)).astype(np.float32)
    out = np.where(big, np.float32(np.inf), out).astype(np.float32)
    return torch.from_numpy(out)


_LN2_F64 = 0.6931471805599453
_SQRT_HALF_F64 = 0.7071067811865476


def log_det(v: torch.Tensor) -> torch.Tensor:
    """Natural log of positive fp32 ``v`` computed in fp64 from + - * / only,
    returned rounded to fp32.  ``v = m * 2^e`` with ``m`` in [sqrt(1/2), sqrt(2))``;
    ``log m = 2 s (1 + s^2/3 + ... + s^18/19)``, ``s = (m-1)/(m+1)``.
    """
    a = v.detach().to(torch.float64).numpy()
    m, e = np.frexp(a)  # m in [0.5, 1)
    low = m < _SQRT_HALF_F64
    m = np.where(low, m * 2.0, m)
    e = np.where(low, e - 1, e).astype(np.float64)
    s = (m - 1.0) / (m + 1.0)
    s2 = s * s
    p = np.full_like(s, 1.0 / 19.0)
    for d in (17.0, 15.0, 13.0, 11.0, 9.0, 7.0, 5.0, 3.0, 1.0):
        p = p * s2
        p = p + (1.0 / d)
    r = (2.0 * s) * p
    r = r + e * _LN2_F64
    return torch.from_numpy(r.astype(np.float32))


# --------------------------------------------------------------------------
# RMSNorm (+ residual) with an integer sum of squares
# --------------------------------------------------------------------------

def rms_norm(
    x: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    residual: torch.Tensor | None = None,
    frac_bits: int = 16,
) -> tuple[torch.Tensor, torch.Tensor | None]:
    """RMSNorm following ``fxpr_vllm/_triton/rms_norm.py:38-64`` except that the
    sum of squares is ``sum(float_to_fixed(r*r, Q.frac, int64))`` summed as
    integers, so it does not depend on the reduction order or block size.

    Returns ``(y, new_residual)``; the residual is rounded to the IO dtype
    before the second pass (rms_norm.py:44-48, 58-61).
    """
    dt = x.dtype
    h = x.shape[-1]
    xf = x.reshape(-1, h).to(torch.float32)
    new_res = None
    if residual is not None:
        xf = xf + residual.reshape(-1, h).to(torch.float32)
        new_res = xf.to(dt)
        x2 = new_res.to(torch.float32)
    else:
        x2 = xf
    sq = xf * xf
    acc = float_to_fixed(sq, 64, frac_bits).sum(dim=-1, keepdim=True)
    # The per-row scalar chain runs in numpy: its float32 divide and sqrt are
    # correctly rounded, whereas torch's vectorised CPU sqrt is not (a few results
    # per thousand are off by one ulp) and torch divides by a scalar as x * (1/s).
    total = (acc.to(torch.float32) * (1.0 / float(1 << frac_bits))).numpy()
    mean = np.maximum(total / np.float32(h), np.float32(0.0)).astype(np.float32)
    rrms_np = (np.float32(1.0) / np.sqrt((mean + np.float32(eps)).astype(np.float32))).astype(np.float32)
    rrms = torch.from_numpy(rrms_np)
    y = (x2 * weight.to(torch.float32)) * rrms
    y = y.to(dt).reshape(x.shape)
    if new_res is not None:
        new_res = new_res.reshape(x.shape)
    return y, new_res


# --------------------------------------------------------------------------
# Log-softmax with an integer sum of exponentials (no reference counterpart)
# --------------------------------------------------------------------------

def log_softmax(x: torch.Tensor, frac_bits: int = 16) -> torch.Tensor:
    """``out_i = (x_i - m) - log(sum_i Q(exp(x_i - m)))`` over the last dim.

    ``m`` is the exact row maximum, ``exp(d) = exp2_det(d * log2(e))``, the sum
    runs over int64 Q-format integers, ``log`` is :func:`log_det`.  Output fp32.
    """
    xf = x.to(torch.float32)
    m = xf.max(dim=-1, keepdim=True).values
    d = xf - m
    t = d * torch.tensor(RCP_LN2, dtype=torch.float32)
    e = exp2_det(t)
    s = float_to_fixed(e, 64, frac_bits).sum(dim=-1, keepdim=True)
    sf = s.to(torch.float32) * (1.0 / float(1 << frac_bits))
    return d - log_det(sf)


# --------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------

def gemm_int_from_partials(
    partials: torch.Tensor, int_bits: int, frac_bits: int
) -> torch.Tensor:
    """Integer stage of the GEMM given the fp32 per-K-tile partials ``[T, M, N]``:
    quantise each, add as integers (wrapping in the accumulator width);
    gemm.py:189-190.  Returns int64 holding the ``int_bits``-wide value."""
    acc = torch.zeros(partials.shape[1:], dtype=torch.int64)
    for t in range(partials.shape[0]):
        acc = acc + float_to_fixed(partials[t], int_bits, frac_bits).to(torch.int64)
        acc = _wrap_to_bits(acc, int_bits)
    return acc


def gemm_epilogue(
    acc: torch.Tensor, bias: torch.Tensor | None, out_dtype: torch.dtype, frac_bits: int
) -> torch.Tensor:
    """``T(fp32(acc) * 2^-frac + fp32(bias))``; gemm.py:195-204."""
    c = acc.to(torch.float32) * (1.0 / float(1 << frac_bits))
    if bias is not None:
        c = c + bias.to(torch.float32)[None, :]
    return c.to(out_dtype)


def gemm_partials(
    a: torch.Tensor, b: torch.Tensor, k_tile: int, sequential: bool = False
) -> torch.Tensor:
    """fp32 partial products per K-tile, ``[T, M, N]`` (K tail zero-padded,
    gemm.py:185-187).

    ``sequential=True`` adds the products one ``k`` at a time in ascending order
    with separate fp32 multiply and add -- the exact order of the portable CUDA
    kernel; ``False`` uses a CPU fp32 matmul (tensor-core stand-in, last-ulp
    differences expected)."""
    af = a.to(torch.float32)
    bf = b.to(torch.float32)
    m, k = af.shape
    n = bf.shape[1]
    tiles = max(1, -(-k // k_tile)) if k > 0 else 0
    out = torch.zeros((tiles, m, n), dtype=torch.float32)
    for t in range(tiles):
        lo, hi = t * k_tile, min(k, (t + 1) * k_tile)
        if sequential:
            p = torch.zeros((m, n), dtype=torch.float32)
            for kk in range(lo, hi):
                p = p + af[:, kk : kk + 1] * bf[kk : kk + 1, :]
            out[t] = p
        else:
            out[t] = af[:, lo:hi] @ bf[lo:hi, :]
    return out


def gemm_fxp(
    a: torch.Tensor,
    b: torch.Tensor,
    bias: torch.Tensor | None,
    int_bits: int,
    frac_bits: int,
    k_tile: int | None = None,
    sequential: bool = False,
    return_int: bool = False,
):
    """Full fixed-point GEMM; gemm.py:123-204."""
    kt = k_tile or GEMM_BLOCK_K[a.dtype]
    acc = gemm_int_from_partials(gemm_partials(a, b, kt, sequential), int_bits, frac_bits)
    if return_int:
        return acc
    return gemm_epilogue(acc, bias, a.dtype, frac_bits)


# --------------------------------------------------------------------------
# Paged attention
# --------------------------------------------------------------------------

def _seq_dot_rows(q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
    """``q [R, D] . k [N, D]`` -> ``[R, N]`` adding d = 0, 1, ... in order."""
    s = torch.zeros((q.shape[0], k.shape[0]), dtype=torch.float32)
    for d in range(q.shape[1]):
        s = s + q[:, d : d + 1] * k[:, d][None, :]
    return s


def attention_fxp(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    query_start_loc: torch.Tensor,
    seq_lens: torch.Tensor,
    block_table: torch.Tensor,
    *,
    alibi_slopes: torch.Tensor | None = None,
    is_causal: bool = True,
    softmax_scale: float | None = None,
    int_bits: int = 32,
    frac_bits: int = 16,
    logit_softcap: float = 0.0,
    window_size: int = 0,
    sequential: bool = True,
    exp2_fn=None,
    return_int: bool = False,
):
    """Unified prefill+decode paged attention, one query row at a time;
    attention.py:103-121 (score post-processing), :199-215 (masks),
    :233-301 (two passes, integer denominator and numerator).

    Key tiles are ``BLOCK_N`` wide starting at key 0 (no sliding window) so the
    per-tile P.V partials that get quantised are the same for any batching or
    split count.  ``sequential=True`` mirrors the portable CUDA kernel's
    summation order exactly (d ascending for scores, key ascending for P.V).
    Sliding windows are evaluated per query row (``lo`` = the row's own first
    visible key rounded to nothing: tiles start at 0), a deliberate
    simplification of attention.py:199-206 that keeps tile boundaries
    batch-invariant; rows see exactly the same keys.
    """
    dt = q.dtype
    block_n = ATTN_BLOCK_N[dt]
    t_q, hq, d = q.shape
    page = kv_cache.shape[2]
    hkv = kv_cache.shape[3]
    group = hq // hkv
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    ss_log2 = np.float32(float(scale) * RCP_LN2)
    cap2 = np.float32(float(logit_softcap) * RCP_LN2)
    exp2 = exp2_fn or exp2_det
    out = torch.zeros_like(q)
    int_denom = torch.zeros((t_q, hq), dtype=torch.int64)
    int_wv = torch.zeros((t_q, hq, d), dtype=torch.int64)
    inv = 1.0 / float(1 << frac_bits)
    qsl = query_start_loc.tolist()
    for r, seq_len in enumerate(seq_lens.tolist()):
        q0, q1 = qsl[r], qsl[r + 1]
        q_len = q1 - q0
        if q_len <= 0:
            continue
        ctx = seq_len - q_len
        pos = torch.arange(seq_len)
        phys = block_table[r, pos // page].long()
        k_all = kv_cache[phys, 0, pos % page]  # [S, Hkv, D]
        v_all = kv_cache[phys, 1, pos % page]
        for h in range(hq):
            kh = k_all[:, h // group].to(torch.float32)
            vh = v_all[:, h // group].to(torch.float32)
            qh = q[q0:q1, h].to(torch.float32)
            if sequential:
                raw = _seq_dot_rows(qh, kh)
            else:
                raw = qh @ kh.T
            s = raw * torch.tensor(ss_log2)
            if logit_softcap > 0.0:
                s = torch.tensor(cap2) * torch.tanh(s / torch.tensor(cap2))
            rows = ctx + torch.arange(q_len)
            if alibi_slopes is not None:
                s = s + alibi_slopes[h].to(torch.float32) * (
                    pos[None, :].to(torch.float32) - rows[:, None].to(torch.float32)
                )
            valid = torch.ones((q_len, seq_len), dtype=torch.bool)
            if is_causal:
                valid &= pos[None, :] < (rows[:, None] + 1)
            if window_size > 0:
                valid &= pos[None, :] >= (rows[:, None] - window_size + 1)
            s = torch.where(valid, s, torch.tensor(float("-inf")))
            gmax = s.max(dim=1).values
            gmax = torch.where(torch.isinf(gmax), torch.zeros_like(gmax), gmax)
            w = exp2(s - gmax[:, None])
            w = torch.where(valid, w, torch.zeros_like(w))
            denom = float_to_fixed(w, int_bits, frac_bits).to(torch.int64).sum(dim=1)
            denom = _wrap_to_bits(denom, int_bits)
            wq = w.to(dt).to(torch.float32)
            wv = torch.zeros((q_len, d), dtype=torch.int64)
            for lo in range(0, seq_len, block_n):
                hi = min(seq_len, lo + block_n)
                if sequential:
                    pv = torch.zeros((q_len, d), dtype=torch.float32)
                    for j in range(lo, hi):
                        pv = pv + wq[:, j : j + 1] * vh[j][None, :]
                else:
                    pv = wq[:, lo:hi] @ vh[lo:hi]
                wv = _wrap_to_bits(
                    wv + float_to_fixed(pv, int_bits, frac_bits).to(torch.int64), int_bits
                )
            int_denom[q0:q1, h] = denom
            int_wv[q0:q1, h] = wv
            den = torch.clamp(denom.to(torch.float32) * inv, min=1.0e-6)
            num = wv.to(torch.float32) * inv
            out[q0:q1, h] = (num / den[:, None]).to(dt)
    if return_int:
        return out, int_denom, int_wv
    return out


# --------------------------------------------------------------------------
# Tensor-parallel row-parallel reduce (no reference counterpart)
# --------------------------------------------------------------------------

def tp_row_parallel(
    a: torch.Tensor,
    b: torch.Tensor,
    bias: torch.Tensor | None,
    tp: int,
    int_bits: int,
    frac_bits: int,
    k_tile: int | None = None,
    sequential: bool = False,
) -> torch.Tensor:
    """Shard K over ``tp`` ranks, sum the ranks' integer accumulators, convert
    once.  Equals :func:`gemm_fxp` whenever K/tp is a whole number of K-tiles."""
    k = a.shape[1]
    assert k % tp == 0
    ks = k // tp
    acc = torch.zeros((a.shape[0], b.shape[1]), dtype=torch.int64)
    for r in range(tp):
        acc = acc + gemm_fxp(
            a[:, r * ks : (r + 1) * ks], b[r * ks : (r + 1) * ks], None,
            int_bits, frac_bits, k_tile, sequential, return_int=True,
        )
        acc = _wrap_to_bits(acc, int_bits)
    return gemm_epilogue(acc, bias, a.dtype, frac_bits)
