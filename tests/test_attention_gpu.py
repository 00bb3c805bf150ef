"""GPU parity of the unified paged attention.

* CUDA-core route: bit-exact against the CPU oracle.
* default route: within tolerance of the oracle / float softmax, and bitwise
  invariant to the KV split count, repeats and batching (decode row == the same
  row computed inside a prefill chunk).
* the reference's tests (fxpr_vllm/_tests/test_decode.py, test_prefill.py)
  re-stated, including its page_size=1 adapter.
"""
from __future__ import annotations

import math

import pytest
import torch

import fxpr_vllm  # noqa: F401
from fxpr_vllm import _lib as L
from oracle import fxp_oracle as orc

pytestmark = pytest.mark.gpu
_DTYPES = [torch.float16, torch.bfloat16, torch.float32]


def _h():
    import fxp_helpers
    return fxp_helpers


def _mixed_batch(dtype, hq, hkv, d, page, seed, ctx=(37, 150, 70), qlens=(1, 5, 70)):
    g = torch.Generator().manual_seed(seed)
    seq = list(ctx)  # seq_lens count the new tokens too
    kv, bt = _h().make_paged_kv(seq, hkv, d, page, dtype, g)
    qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32)
    q = torch.randn((int(qsl[-1]), hq, d), generator=g).to(dtype)
    return q.cuda(), kv, qsl.cuda(), torch.tensor(seq, dtype=torch.int32).cuda(), bt, max(qlens)


@pytest.mark.parametrize("dtype", _DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 32, 16), (4, 1, 80, 16), (2, 2, 64, 1)])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("int_bits", [32, 64])
def test_portable_bit_exact(dtype, hq, hkv, d, page, splits, int_bits):
    q, kv, qsl, sl, bt, mq = _mixed_batch(dtype, hq, hkv, d, page, 7)
    with L.overrides(attn_portable=True):
        got = _h().run_attention(q, kv, qsl, sl, bt, mq, int_bits=int_bits, splits=splits).cpu()
    exp = orc.attention_fxp(q.cpu(), kv.cpu(), qsl.cpu(), sl.cpu(), bt.cpu(), int_bits=int_bits)
    assert torch.equal(got.view(torch.uint8), exp.view(torch.uint8))


@pytest.mark.parametrize("kwargs", [dict(causal=False), dict(window=24), dict(alibi=True),
                                    dict(scale=0.05), dict(frac_bits=8)])
def test_portable_flags_bit_exact(kwargs):
    dtype = torch.bfloat16
    q, kv, qsl, sl, bt, mq = _mixed_batch(dtype, 4, 2, 32, 16, 9)
    kw = dict(kwargs)
    alibi = None
    if kw.pop("alibi", False):
        alibi = torch.tensor([0.1, 0.2, 0.3, 0.4]) * orc.RCP_LN2
    with L.overrides(attn_portable=True):
        got = _h().run_attention(q, kv, qsl, sl, bt, mq, splits=2,
                                 alibi=None if alibi is None else alibi.cuda(), **kw).cpu()
    exp = orc.attention_fxp(q.cpu(), kv.cpu(), qsl.cpu(), sl.cpu(), bt.cpu(),
                            alibi_slopes=alibi, is_causal=kw.get("causal", True),
                            softmax_scale=kw.get("scale"), frac_bits=kw.get("frac_bits", 16),
                            window_size=kw.get("window", 0))
    assert torch.equal(got.view(torch.uint8), exp.view(torch.uint8))


def _float_attention(q, kv, qsl, sl, bt, causal=True, softcap=0.0):
    q, kv = q.float().cpu(), kv.float().cpu()
    out = torch.zeros_like(q)
    page, hkv = kv.shape[2], kv.shape[3]
    hq, d = q.shape[1], q.shape[2]
    for r in range(sl.numel()):
        s = int(sl[r]); q0, q1 = int(qsl[r]), int(qsl[r + 1])
        pos = torch.arange(s)
        k = kv[bt[r, pos // page].long().cpu(), 0, pos % page]
        v = kv[bt[r, pos // page].long().cpu(), 1, pos % page]
        rows = s - (q1 - q0) + torch.arange(q1 - q0)
        for h in range(hq):
            sc = (q[q0:q1, h] @ k[:, h // (hq // hkv)].T) / math.sqrt(d)
            if softcap > 0:
                sc = softcap * torch.tanh(sc / softcap)
            if causal:
                sc = sc.masked_fill(pos[None, :] > rows[:, None], float("-inf"))
            out[q0:q1, h] = torch.softmax(sc, -1) @ v[:, h // (hq // hkv)]
    return out


@pytest.mark.parametrize("dtype", _DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 32, 16), (32, 8, 128, 16), (8, 8, 64, 32)])
@pytest.mark.parametrize("causal", [True, False])
def test_default_route_vs_float_softmax(dtype, hq, hkv, d, page, causal):
    q, kv, qsl, sl, bt, mq = _mixed_batch(dtype, hq, hkv, d, page, 11, ctx=(200, 64, 129),
                                          qlens=(1, 64, 33))
    got = _h().run_attention(q, kv, qsl, sl, bt, mq, causal=causal).float().cpu()
    ref = _float_attention(q, kv, qsl, sl, bt, causal)
    assert torch.allclose(got, ref, atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_default_route_close_to_oracle(dtype):
    q, kv, qsl, sl, bt, mq = _mixed_batch(dtype, 8, 2, 128, 16, 13, ctx=(300, 90), qlens=(1, 40))
    got = _h().run_attention(q, kv, qsl, sl, bt, mq, int_bits=64).float().cpu()
    exp = orc.attention_fxp(q.cpu(), kv.cpu(), qsl.cpu(), sl.cpu(), bt.cpu(), int_bits=64,
                            sequential=False, exp2_fn=torch.exp2).float()
    # outputs agree to one rounding step of the IO dtype plus a couple of Q16.16 LSB
    tol = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -9
    assert (got - exp).abs().max().item() <= tol


@pytest.mark.parametrize("dtype", _DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 32, 16), (32, 8, 128, 16)])
@pytest.mark.parametrize("int_bits", [32, 64])
def test_split_and_repeat_invariance(dtype, hq, hkv, d, page, int_bits):
    q, kv, qsl, sl, bt, mq = _mixed_batch(dtype, hq, hkv, d, page, 17, ctx=(160, 96, 700),
                                          qlens=(1, 1, 1))
    ref = _h().run_attention(q, kv, qsl, sl, bt, 1, int_bits=int_bits, splits=1)
    for splits in (1, 2, 4, 8, 16):
        for _ in range(2):
            got = _h().run_attention(q, kv, qsl, sl, bt, 1, int_bits=int_bits, splits=splits)
            assert torch.equal(ref, got), f"splits={splits}"


@pytest.mark.parametrize("dtype", _DTYPES)
def test_prefill_split_invariance_and_auto_policy(dtype):
    q, kv, qsl, sl, bt, mq = _mixed_batch(dtype, 4, 2, 64, 16, 19, ctx=(130, 257), qlens=(130, 257))
    ref = _h().run_attention(q, kv, qsl, sl, bt, mq, splits=1)
    for splits in (0, 2, 4, 8):
        assert torch.equal(ref, _h().run_attention(q, kv, qsl, sl, bt, mq, splits=splits))


@pytest.mark.parametrize("dtype", _DTYPES)
@pytest.mark.parametrize("hq,hkv,d", [(4, 2, 32), (32, 8, 128)])
def test_decode_row_equals_prefill_row(dtype, hq, hkv, d):
    """Batch invariance across kernel variants: the last token of a prefill chunk
    and the same token issued as a decode step give identical bits."""
    g = torch.Generator().manual_seed(23)
    s = 173
    kv, bt = _h().make_paged_kv([s], hkv, d, 16, dtype, g)
    q = torch.randn((s, hq, d), generator=g).to(dtype).cuda()
    sl = torch.tensor([s], dtype=torch.int32).cuda()
    full = _h().run_attention(q, kv, torch.tensor([0, s], dtype=torch.int32).cuda(), sl, bt, s)
    chunk = _h().run_attention(q[-40:].contiguous(), kv, torch.tensor([0, 40], dtype=torch.int32).cuda(), sl, bt, 40)
    dec = _h().run_attention(q[-1:].contiguous(), kv, torch.tensor([0, 1], dtype=torch.int32).cuda(), sl, bt, 1)
    assert torch.equal(full[-1], dec[0]) and torch.equal(full[-40:], chunk)


def test_key_tile_permutation_invariance_page1():
    """Reference's test_prefill.py:246-279 idea: permuting whole 64-key tiles of a
    non-causal problem leaves the output bits unchanged."""
    dtype, hq, d, n = torch.bfloat16, 2, 32, 256
    g = torch.Generator().manual_seed(29)
    q = torch.randn((n, hq, d), generator=g).to(dtype).cuda()
    k = torch.randn((n, hq, d), generator=g).to(dtype)
    v = torch.randn((n, hq, d), generator=g).to(dtype)

    def run(kk, vv):
        kv = torch.stack([kk, vv], dim=1).unsqueeze(2).contiguous().cuda()  # page_size 1
        bt = torch.arange(n, dtype=torch.int32).reshape(1, n).cuda()
        return _h().run_attention(q, kv, torch.tensor([0, n], dtype=torch.int32).cuda(),
                                  torch.tensor([n], dtype=torch.int32).cuda(), bt, n, causal=False)

    tperm = torch.randperm(4, generator=g)
    idx = torch.cat([torch.arange(t * 64, (t + 1) * 64) for t in tperm])
    assert torch.equal(run(k, v), run(k[idx], v[idx]))


def test_softcap_and_errors():
    q, kv, qsl, sl, bt, mq = _mixed_batch(torch.bfloat16, 4, 2, 32, 16, 31)
    got = _h().run_attention(q, kv, qsl, sl, bt, mq, softcap=20.0).float().cpu()
    ref = _float_attention(q, kv, qsl, sl, bt, True, softcap=20.0)
    assert torch.allclose(got, ref, atol=5e-2, rtol=5e-2)
    o = torch.empty_like(q)
    with pytest.raises(TypeError):
        torch.ops.fxpr.unified_attention_fxp(q, kv, o, qsl.long(), sl, bt, mq, None, True, None, 32, 16, 0.0, 0, 1)
    with pytest.raises(ValueError):
        torch.ops.fxpr.unified_attention_fxp(q, kv[:, :1], o, qsl, sl, bt, mq, None, True, None, 32, 16, 0.0, 0, 1)
    with pytest.raises(ValueError):
        torch.ops.fxpr.unified_attention_fxp(q, kv, o, qsl, sl, bt, mq, None, True, None, 32, 16, 0.0, 0, -1)
    with pytest.raises(TypeError):
        torch.ops.fxpr.unified_attention_fxp(q, kv.float(), o, qsl, sl, bt, mq, None, True, None, 32, 16, 0.0, 0, 1)
    # empty batch is a no-op
    torch.ops.fxpr.unified_attention_fxp(q[:0], kv, o[:0], qsl[:1], sl[:0], bt[:0], 0, None, True, None, 32, 16, 0.0, 0, 1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (8, 8, 64)])
@pytest.mark.parametrize("int_bits,frac_bits", [(64, 16), (32, 16), (64, 8)])
@pytest.mark.parametrize("outliers", [False, True])
def test_fast_conversion_prefill_equals_exact_conversion(dtype, hq, hkv, d, int_bits, frac_bits, outliers):
    """The prefill kernel's second pass converts on the FP32 pipe (magic-number rounding,
    32-bit wrap-around sums, exact fix-up for partials outside its range); the bits must be
    those of the cvt.rni.sat kernel.  Outliers in V push P.V partials past 2^(22-frac)."""
    from fxpr_vllm import _native as nat
    q, kv, qsl, sl, bt, mq = _mixed_batch(dtype, hq, hkv, d, 16, 21, ctx=(300, 150, 70), qlens=(300, 5, 70))
    if outliers:
        kv = kv.clone()
        kv[3::7, 1, 5, :, ::3] = 3000.0 if frac_bits == 16 else 60000.0
        kv[2::5, 1, 9, :, 1::4] = -2500.0
    outs = []
    for flags in (0, nat.ATTN_EXACT_CONVERT):
        with L.overrides(attn_flags=flags):
            outs.append(_h().run_attention(q, kv, qsl, sl, bt, mq, int_bits=int_bits, frac_bits=frac_bits))
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kwargs", [dict(causal=False), dict(window=24), dict(window=100), dict(alibi=True),
                                    dict(scale=0.05), dict(frac_bits=8), dict(softcap=20.0)])
@pytest.mark.parametrize("splits", [1, 3])
def test_tensor_core_route_feature_flags_close_to_oracle(dtype, kwargs, splits):
    """Sliding window, ALiBi, soft-cap, non-causal, custom scale and Q8 on the tensor-core
    kernels (decode and prefill rows in one batch), against the oracle evaluated with the
    same non-sequential partials: one rounding step of the io dtype plus a few Q LSBs; and the
    split count must not change a bit."""
    q, kv, qsl, sl, bt, mq = _mixed_batch(dtype, 8, 2, 128, 16, 17, ctx=(300, 150, 70), qlens=(1, 40, 70))
    kw = dict(kwargs)
    alibi = None
    if kw.pop("alibi", False):
        alibi = torch.linspace(0.05, 0.4, 8) * orc.RCP_LN2
    run = lambda s: _h().run_attention(q, kv, qsl, sl, bt, mq, int_bits=64, splits=s,
                                       alibi=None if alibi is None else alibi.cuda(), **kw)
    got = run(splits)
    assert torch.equal(got.view(torch.int16), run(1).view(torch.int16))
    exp = orc.attention_fxp(q.cpu(), kv.cpu(), qsl.cpu(), sl.cpu(), bt.cpu(), int_bits=64,
                            alibi_slopes=alibi, is_causal=kw.get("causal", True),
                            softmax_scale=kw.get("scale"), frac_bits=kw.get("frac_bits", 16),
                            window_size=kw.get("window", 0), logit_softcap=kw.get("softcap", 0.0),
                            sequential=False, exp2_fn=torch.exp2).float()
    frac = kw.get("frac_bits", 16)
    tol = (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -9) * 2 + 8 * 2.0 ** -frac
    assert (got.float().cpu() - exp).abs().max().item() <= tol * max(1.0, float(exp.abs().max()))


@pytest.mark.parametrize("case", [
    # (seq_lens, q_lens, q heads, kv heads, page, dtype, int_bits, extra arguments)
    ([80, 33], [80, 33], 32, 8, 16, torch.bfloat16, 64, {}),
    ([200, 64, 17], [5, 64, 17], 32, 8, 16, torch.bfloat16, 64, {}),          # chunked prefill + short rows
    ([1000, 333], [1000, 333], 32, 8, 16, torch.bfloat16, 32, {}),
    ([500, 129], [100, 129], 8, 8, 32, torch.float16, 64, {}),                # no GQA, 32-token pages
    ([300, 257], [300, 200], 16, 2, 16, torch.bfloat16, 64, dict(softcap=30.0)),
    ([300, 257], [300, 200], 32, 8, 16, torch.bfloat16, 64, dict(window=100)),
    ([300, 257], [300, 200], 32, 8, 16, torch.bfloat16, 64, dict(causal=False)),
    ([300, 257], [300, 200], 32, 8, 16, torch.bfloat16, 64, dict(alibi=True)),
    ([2100], [2100], 32, 8, 16, torch.bfloat16, 64, {}),
    ([700, 90], [700, 90], 32, 8, 64, torch.bfloat16, 64, {}),                # 64-token pages: one box per tile
    ([700, 90], [300, 90], 32, 8, 128, torch.float16, 32, {}),
])
def test_tcgen05_prefill_kernel_equals_mma_sync_kernel(case):
    """The tcgen05 / tensor-memory prefill kernel against the mma.sync kernel it replaces: a
    tcgen05.mma chain of 16-deep steps gives the same fp32 bits as the mma.sync.m16n8k16 chain,
    every other step is the same instruction, so the outputs are equal bit for bit -- which is
    also what keeps a prefill row equal to the decode step of the same token."""
    from fxpr_vllm import _native as nat
    from fxpr_vllm import synthetic as syn

    sls, qls, hq, hkv, page, dtype, int_bits, kw = case
    kw = dict(kw)
    q, kv, qsl, sl, bt = syn.paged_attention_inputs(sls, qls, q_heads=hq, kv_heads=hkv, head_dim=128, page=page,
                                                    dtype=dtype, seed=100 + len(sls) + hq)
    alibi = None
    if kw.pop("alibi", False):
        alibi = torch.arange(1, hq + 1, device="cuda", dtype=torch.float32) * 0.01 * orc.RCP_LN2
    outs = []
    for flags in (0, nat.ATTN_NO_TCGEN05):
        o = torch.full_like(q, float("nan"))
        with L.overrides(attn_flags=flags):
            torch.ops.fxpr.unified_attention_fxp(q, kv, o, qsl, sl, bt, max(qls), alibi, kw.get("causal", True), None,
                                                 int_bits, 16, kw.get("softcap", 0.0), kw.get("window", 0), 1)
        outs.append(o)
    L.check_device_status()
    assert not outs[0].isnan().any()
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
