"""The allocation-free attention entry point, called straight through the C ABI.

Some hosts of this library cannot allocate device memory on the attention path
(all of HBM already belongs to the KV cache, there is no torch allocator, or a
cudaMalloc stall is not acceptable), so ``fxpr_attention_static_scratch`` keeps
the split path's scratch in a fixed array inside the library.  Only the
CUDA-core route of the attention uses scratch (the tensor-core route merges its
splits inside a thread-block cluster), so these tests force that route
(``ATTN_FORCE_PORTABLE``) or use inputs that always take it (fp32, head size
96).  They check that the entry point gives the same bits as ``fxpr_attention``
with caller-owned scratch on calls in a row that differ in shape and split
count (the array keeps the previous call's contents, so stale counters or
totals would corrupt the next call), and that it refuses problems larger than
the array.  The file name sorts last so a run that stops at the first failure
has already run every other test.
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, q, kv, o, qsl, sl, bt, splits, flags, scratch=None, max_q=1):
    from fxpr_vllm import _native as nat

    k, v = kv.select(1, 0), kv.select(1, 1)
    args = [q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), qsl.data_ptr(), sl.data_ptr(),
            bt.data_ptr(), None, nat.DTYPE_CODE[q.dtype], q.shape[0], sl.shape[0], q.shape[1],
            kv.shape[3], q.shape[2], kv.shape[2], q.stride(0), q.stride(1), o.stride(0), o.stride(1),
            kv.stride(0), kv.stride(2), kv.stride(3), bt.stride(0), max_q, flags,
            1.0 / (q.shape[2] ** 0.5), 0.0, 0, 64, 16, splits]
    stream = torch.cuda.current_stream().cuda_stream
    if fn_name == "fxpr_attention":
        args += [None if scratch is None else scratch.data_ptr(),
                 0 if scratch is None else scratch.numel(), None, stream]
    else:
        args += [None, stream]
    return getattr(lib, fn_name)(*args)


# (context lengths, query lengths, dtype, q heads, kv heads, head size, splits, force the CUDA-core route)
_CASES = [
    ([200, 64, 333, 16], [1, 1, 1, 1], torch.bfloat16, 32, 8, 128, 4, True),
    ([90, 150], [3, 1], torch.float32, 8, 2, 64, 8, False),          # fp32 always takes the CUDA-core route
    ([120, 40, 77], [1, 2, 1], torch.float16, 6, 2, 96, 2, False),   # so does head size 96
    ([257, 31], [1, 1], torch.bfloat16, 32, 8, 128, 16, True),
]


def test_static_scratch_matches_caller_scratch_on_calls_in_a_row():
    import fxpr_vllm  # noqa: F401
    from fxpr_vllm import _native as nat
    from fxpr_vllm import synthetic as syn

    lib = nat.load()
    cap = lib.fxpr_attention_static_scratch_capacity()
    assert cap == 4 << 20
    for rnd in range(2):                 # the second round meets the array as the first one left it
        for n, (lens, qlens, dtype, hq, hkv, d, splits, force) in enumerate(_CASES):
            q, kv, qsl, sl, bt = syn.paged_attention_inputs(lens, qlens, q_heads=hq, kv_heads=hkv, head_dim=d, dtype=dtype,
                                                            seed=50 + n)
            flags = nat.ATTN_CAUSAL | (nat.ATTN_FORCE_PORTABLE if force else 0)
            need = lib.fxpr_attention_scratch_bytes(q.shape[0], hq, d, 64, splits)
            assert 0 < need <= cap
            scratch = torch.empty(need, device="cuda", dtype=torch.uint8)
            o_ref = torch.empty_like(q)
            assert _call(lib, "fxpr_attention", q, kv, o_ref, qsl, sl, bt, splits, flags, scratch,
                         max(qlens)) == 0
            for _ in range(2):           # twice in a row on the same problem as well
                o = torch.full_like(q, float("nan"))
                assert _call(lib, "fxpr_attention_static_scratch", q, kv, o, qsl, sl, bt, splits, flags,
                             max_q=max(qlens)) == 0
                torch.cuda.synchronize()
                assert torch.equal(o, o_ref), (rnd, n)
            # one split needs no scratch at all
            o1 = torch.empty_like(q)
            assert _call(lib, "fxpr_attention_static_scratch", q, kv, o1, qsl, sl, bt, 1, flags,
                         max_q=max(qlens)) == 0
            torch.cuda.synchronize()
            assert torch.equal(o1, o_ref)


def test_static_scratch_refuses_oversized_problems_on_the_route_that_needs_it():
    import fxpr_vllm  # noqa: F401
    from fxpr_vllm import _native as nat
    from fxpr_vllm import synthetic as syn

    lib = nat.load()
    lens = [32] * 512      # 512 tokens x 32 heads x 128 dims x 8 B > 4 MiB
    q, kv, qsl, sl, bt = syn.paged_attention_inputs(lens, [1] * len(lens), seed=43)
    assert lib.fxpr_attention_scratch_bytes(q.shape[0], 32, 128, 64, 2) > lib.fxpr_attention_static_scratch_capacity()
    o = torch.zeros_like(q)
    rc = _call(lib, "fxpr_attention_static_scratch", q, kv, o, qsl, sl, bt, 2,
               nat.ATTN_CAUSAL | nat.ATTN_FORCE_PORTABLE)
    assert rc == nat.FXPR_ERR_SCRATCH
    assert b"built-in" in lib.fxpr_last_error()
    torch.cuda.synchronize()
    assert not o.any()      # nothing was launched
    # the same problem on the tensor-core route uses no scratch, so it is served whatever its size
    o_ref = torch.empty_like(q)
    scratch = torch.empty(lib.fxpr_attention_scratch_bytes(q.shape[0], 32, 128, 64, 2), device="cuda",
                          dtype=torch.uint8)
    assert _call(lib, "fxpr_attention", q, kv, o_ref, qsl, sl, bt, 2, nat.ATTN_CAUSAL, scratch) == 0
    assert _call(lib, "fxpr_attention_static_scratch", q, kv, o, qsl, sl, bt, 2, nat.ATTN_CAUSAL) == 0
    torch.cuda.synchronize()
    assert torch.equal(o, o_ref)
