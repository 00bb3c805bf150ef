"""``torch.ops.fxpr.*`` schemas and their CUDA implementations.

The six schema strings are those of ``fxpr_vllm/_lib.py:15-33`` in the
reference, so vLLM-side code written against the reference keeps working.
Implementations are registered for the CUDA dispatch key only (CPU tensors get
the dispatcher's ``NotImplementedError``, as with the reference) and hand raw
pointers plus the current stream to the C ABI in ``libfxpr_b200.so``.

Three ops are additions with no counterpart in the reference:
``log_softmax_fxp`` (order-free sampler log-softmax), ``gemm_fxp_int`` and
``gemm_fxp_epilogue`` (integer accumulators out / back in, for the
tensor-parallel integer all-reduce).
"""
from __future__ import annotations

import contextlib
import math
import threading

import torch

from . import _native as nat
from .config import get_runtime_config

_lib = torch.library.Library("fxpr", "DEF")

_lib.define("float_to_fixed(Tensor x, int int_bits, int fxp_frac_bits) -> Tensor")
_lib.define("fixed_to_float(Tensor x, int float_bits, int fxp_frac_bits) -> Tensor")
_lib.define("rms_norm_fxp(Tensor x, Tensor weight_fp32, float eps) -> Tensor")
_lib.define(
    "rms_norm_fxp_residual(Tensor x, Tensor(a!) residual, Tensor weight_fp32, "
    "float eps) -> Tensor"
)
_lib.define(
    "gemm_fxp(Tensor a, Tensor b, Tensor? bias, int fxp_int_bits, "
    "int fxp_frac_bits) -> Tensor"
)
_lib.define(
    "unified_attention_fxp(Tensor q, Tensor kv_cache, Tensor(a!) o, "
    "Tensor query_start_loc, Tensor seq_lens, Tensor block_table, "
    "int max_query_len, Tensor? alibi_slopes, bool is_causal, "
    "float? softmax_scale, int fxp_int_bits, int fxp_frac_bits, "
    "float logit_softcap, int window_size, int num_kv_splits) -> ()"
)
# additions
_lib.define("log_softmax_fxp(Tensor x, int fxp_frac_bits) -> Tensor")
_lib.define("rms_norm_fxp_from_int(Tensor acc, Tensor(a!) residual, Tensor weight, Tensor? bias, float eps, "
            "int gemm_frac_bits) -> Tensor")
_lib.define("gemm_fxp_int(Tensor a, Tensor b, int fxp_int_bits, int fxp_frac_bits) -> Tensor")
_lib.define(
    "gemm_fxp_epilogue(Tensor c_int, Tensor? bias, ScalarType out_dtype, "
    "int fxp_frac_bits) -> Tensor"
)

_INT_DTYPE = {16: torch.int16, 32: torch.int32, 64: torch.int64}
_INT_BITS = {v: k for k, v in _INT_DTYPE.items()}
_FLOAT_DTYPE = {16: torch.float16, 32: torch.float32, 64: torch.float64}

_CAST_FLOAT_DTYPES = (torch.float16, torch.float32, torch.float64)  # casts.py:14
_IO_DTYPES = (torch.float32, torch.float16, torch.bfloat16)

# K-tile = determinism granularity per dtype (gemm.py:26-30 of the reference);
# tests read this the way the reference's test reads _BLOCK_K_BY_DTYPE.
BLOCK_K_BY_DTYPE = {torch.float16: 128, torch.bfloat16: 128, torch.float32: 64}
# key-tile width of the attention kernels (attention.py:32-36)
BLOCK_N_BY_DTYPE = {torch.float16: 64, torch.bfloat16: 64, torch.float32: 32}


def _check_frac_bits(n: int) -> None:
    if int(n) not in (8, 16, 32):
        raise ValueError(f"fxp_frac_bits must be 8/16/32, got {n}")


def _check_int_bits(n: int) -> None:
    if int(n) not in (16, 32, 64):
        raise ValueError(f"int_bits must be 16/32/64, got {n}")


@contextlib.contextmanager
def _on_device(t: torch.Tensor):
    """Make ``t``'s device current for the duration of a C call."""
    if t.device.index is not None and t.device.index != torch.cuda.current_device():
        with torch.cuda.device(t.device):
            yield
    else:
        yield


# --------------------------------------------------------------------------
# test / tuning overrides (the public schemas carry no such arguments)
# --------------------------------------------------------------------------

class _Overrides(threading.local):
    gemm_k_tile: int | None = None
    gemm_split_k: int | None = None
    gemm_portable: bool = False
    attn_portable: bool = False
    gemm_partials: bool = False
    gemm_flags: int = 0
    attn_flags: int = 0
    last_partials: torch.Tensor | None = None


_ovr = _Overrides()


@contextlib.contextmanager
def overrides(*, gemm_k_tile=None, gemm_split_k=None, gemm_portable=None,
              attn_portable=None, gemm_partials=None, gemm_flags=None, attn_flags=None):
    """Temporarily pin kernel-selection knobs (K-tile, split-K, portable route)."""
    names = ("gemm_k_tile", "gemm_split_k", "gemm_portable", "attn_portable", "gemm_partials",
             "gemm_flags", "attn_flags")
    vals = (gemm_k_tile, gemm_split_k, gemm_portable, attn_portable, gemm_partials, gemm_flags,
            attn_flags)
    old = {n: getattr(_ovr, n) for n in names}
    try:
        for n, v in zip(names, vals):
            if v is not None:
                setattr(_ovr, n, v)
        yield _ovr
    finally:
        for n, v in old.items():
            setattr(_ovr, n, v)


@contextlib.contextmanager
def static_weights():
    """Inside this block every GEMM's ``b`` operand is a model weight: complete long before the
    launch and not written by any kernel in flight.  The decode-shape GEMM then requests its
    first weight tiles before it waits for the previous kernel of the stream
    (``FXPR_GEMM_WEIGHTS_STATIC``).  Results do not change."""
    old = _ovr.gemm_flags
    _ovr.gemm_flags = int(old) | nat.GEMM_WEIGHTS_STATIC
    try:
        yield
    finally:
        _ovr.gemm_flags = old


# --------------------------------------------------------------------------
# casts
# --------------------------------------------------------------------------

def float_to_fixed_run(x: torch.Tensor, int_bits: int, fxp_frac_bits: int) -> torch.Tensor:
    """casts.py:57-89 of the reference."""
    if not x.is_cuda:
        raise RuntimeError("float_to_fixed: input must be CUDA")
    if x.dtype not in _CAST_FLOAT_DTYPES:
        raise TypeError(
            f"float_to_fixed: unsupported input dtype {x.dtype}; "
            f"expected one of {_CAST_FLOAT_DTYPES}"
        )
    if int_bits not in _INT_DTYPE:
        raise ValueError(f"int_bits must be 16/32/64, got {int_bits}")
    if not (0 <= fxp_frac_bits < 64):
        raise ValueError(f"frac_bits must satisfy 0 <= N < 64, got {fxp_frac_bits}")
    x_c = x.contiguous()
    y = torch.empty_like(x_c, dtype=_INT_DTYPE[int_bits])
    n = x_c.numel()
    if n == 0:
        return y
    with _on_device(x_c):
        st = nat.load().fxpr_float_to_fixed(
            x_c.data_ptr(), nat.DTYPE_CODE[x_c.dtype], y.data_ptr(), int_bits,
            fxp_frac_bits, n, nat.stream_ptr(x_c.device))
    nat.check(st, "float_to_fixed")
    return y


def fixed_to_float_run(x: torch.Tensor, float_bits: int, fxp_frac_bits: int) -> torch.Tensor:
    """casts.py:92-126 of the reference."""
    if not x.is_cuda:
        raise RuntimeError("fixed_to_float: input must be CUDA")
    if x.dtype not in _INT_BITS:
        raise TypeError(
            f"fixed_to_float: unsupported input dtype {x.dtype}; "
            f"expected one of {tuple(_INT_BITS)}"
        )
    if float_bits not in _FLOAT_DTYPE:
        raise ValueError(f"float_bits must be 16/32/64, got {float_bits}")
    if not (0 <= fxp_frac_bits < 64):
        raise ValueError(f"fxp_frac_bits must satisfy 0 <= N < 64, got {fxp_frac_bits}")
    x_c = x.contiguous()
    y = torch.empty_like(x_c, dtype=_FLOAT_DTYPE[float_bits])
    n = x_c.numel()
    if n == 0:
        return y
    with _on_device(x_c):
        st = nat.load().fxpr_fixed_to_float(
            x_c.data_ptr(), _INT_BITS[x_c.dtype], y.data_ptr(), float_bits,
            fxp_frac_bits, n, nat.stream_ptr(x_c.device))
    nat.check(st, "fixed_to_float")
    return y


# --------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------

def _rms_norm_launch(x, w, residual, eps):
    """rms_norm.py:78-134 of the reference (same checks, same contiguity rules)."""
    if not x.is_cuda or not w.is_cuda:
        raise RuntimeError("rms_norm: x and w must be CUDA")
    if x.dtype not in _IO_DTYPES:
        raise TypeError(
            f"rms_norm: unsupported input dtype {x.dtype}; expected one of {_IO_DTYPES}"
        )
    if w.dtype != x.dtype:
        raise TypeError("rms_norm: weight dtype must match input dtype")
    if residual is not None:
        if not residual.is_cuda:
            raise RuntimeError("rms_norm: residual must be CUDA")
        if residual.dtype != x.dtype:
            raise TypeError("rms_norm: residual dtype must match input dtype")
        if residual.shape != x.shape:
            raise ValueError("rms_norm: residual shape must match x")

    hidden = x.shape[-1]
    x_2d = x.reshape(-1, hidden).contiguous()
    y_2d = torch.empty_like(x_2d)
    r_storage = None
    if residual is not None:
        r_2d = residual.reshape(-1, hidden)
        r_storage = r_2d if r_2d.is_contiguous() else r_2d.contiguous()
    rows = x_2d.shape[0]
    if rows > 0 and hidden > 0:
        w_c = w.contiguous()
        with _on_device(x_2d):
            st = nat.load().fxpr_rms_norm(
                x_2d.data_ptr(), nat.ptr(r_storage), w_c.data_ptr(), y_2d.data_ptr(),
                nat.DTYPE_CODE[x.dtype], rows, hidden, float(eps),
                get_runtime_config().fxp_frac_bits, nat.stream_ptr(x.device))
        nat.check(st, "rms_norm")
    if residual is not None and r_storage.data_ptr() != residual.data_ptr():
        residual.copy_(r_storage.view_as(residual))
    return y_2d.view_as(x)


def rms_norm_fxp_from_int_run(acc, residual, w, bias, eps, gemm_frac_bits):
    """Integer accumulators of a row-parallel GEMM (after the cross-rank integer sum) ->
    GEMM epilogue + residual add + RMSNorm in one kernel.  Same bits as
    ``gemm_fxp_epilogue`` followed by ``rms_norm_fxp_residual``."""
    if acc.dtype not in _INT_BITS:
        raise TypeError(f"rms_norm_fxp_from_int: acc must be an integer tensor, got {acc.dtype}")
    if not (acc.is_cuda and residual.is_cuda and w.is_cuda):
        raise RuntimeError("rms_norm_fxp_from_int: tensors must be CUDA")
    if residual.dtype not in _IO_DTYPES or w.dtype != residual.dtype:
        raise TypeError("rms_norm_fxp_from_int: residual and weight must share one io dtype")
    if acc.shape != residual.shape or not (acc.is_contiguous() and residual.is_contiguous()):
        raise ValueError("rms_norm_fxp_from_int: acc and residual must be contiguous and of one shape")
    hidden = residual.shape[-1]
    rows = residual.numel() // hidden if hidden else 0
    y = torch.empty_like(residual)
    if rows and hidden:
        if hidden * 4 > 64 * 1024:
            x = gemm_fxp_epilogue_run(acc.reshape(rows, hidden), bias, residual.dtype, gemm_frac_bits)
            return _rms_norm_launch(x.view_as(residual), w, residual, eps)
        b = None if bias is None else bias.to(residual.dtype).contiguous()
        with _on_device(acc):
            st = nat.load().fxpr_rms_norm_from_int(
                acc.data_ptr(), _INT_BITS[acc.dtype], nat.ptr(b), residual.data_ptr(), w.contiguous().data_ptr(),
                y.data_ptr(), nat.DTYPE_CODE[residual.dtype], rows, hidden, float(eps), int(gemm_frac_bits),
                get_runtime_config().fxp_frac_bits, nat.stream_ptr(acc.device))
        nat.check(st, "rms_norm_fxp_from_int")
    return y


def rms_norm_fxp_run(x, w, eps):
    return _rms_norm_launch(x, w, None, eps)


def rms_norm_fxp_residual_run(x, residual, w, eps):
    return _rms_norm_launch(x, w, residual, eps)


# --------------------------------------------------------------------------
# log-softmax
# --------------------------------------------------------------------------

def log_softmax_fxp_run(x: torch.Tensor, fxp_frac_bits: int) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError("log_softmax_fxp: input must be CUDA")
    if x.dtype not in _IO_DTYPES:
        raise TypeError(f"log_softmax_fxp: unsupported input dtype {x.dtype}")
    cols = x.shape[-1] if x.dim() > 0 else 1
    x_2d = x.reshape(-1, cols).contiguous()
    y = torch.empty(x_2d.shape, device=x.device, dtype=torch.float32)
    if x_2d.numel() > 0:
        with _on_device(x_2d):
            st = nat.load().fxpr_log_softmax(
                x_2d.data_ptr(), nat.DTYPE_CODE[x.dtype], y.data_ptr(), x_2d.shape[0], cols,
                fxp_frac_bits, nat.stream_ptr(x.device))
        nat.check(st, "log_softmax_fxp")
    return y.view(x.shape)


# --------------------------------------------------------------------------
# decoder-layer element-wise steps (no reference counterpart: vLLM ops there)
# --------------------------------------------------------------------------

def rope_kv_write(qkv, cos, sin, positions, seq_ids, block_table, kv_cache, q_heads, kv_heads):
    """Split ``qkv`` [T, (q_heads + 2 kv_heads) * d], rotate Q and K, return Q [T, q_heads, d]
    and write K, V into the paged ``kv_cache`` (num_blocks, 2, page, kv_heads, d)."""
    T = qkv.shape[0]
    d = kv_cache.shape[-1]
    q = torch.empty((T, q_heads, d), device=qkv.device, dtype=qkv.dtype)
    if T == 0:
        return q
    if not (qkv.is_contiguous() and cos.dtype == torch.float32 and sin.dtype == torch.float32
            and positions.dtype == torch.int64 and seq_ids.dtype == torch.int64
            and block_table.dtype == torch.int32 and kv_cache.dtype == qkv.dtype):
        raise TypeError("rope_kv_write: contiguous qkv, fp32 tables, int64 positions / ids, int32 block table")
    with _on_device(qkv):
        st = nat.load().fxpr_rope_kv_write(
            qkv.data_ptr(), nat.DTYPE_CODE[qkv.dtype], cos.data_ptr(), sin.data_ptr(),
            positions.data_ptr(), seq_ids.data_ptr(), block_table.data_ptr(), block_table.stride(0),
            q.data_ptr(), kv_cache.data_ptr(), T, q_heads, kv_heads, d, kv_cache.shape[2],
            kv_cache.stride(0), kv_cache.stride(1), kv_cache.stride(2), kv_cache.stride(3),
            nat.stream_ptr(qkv.device))
    nat.check(st, "rope_kv_write")
    return q


def silu_mul(gate_up):
    """``silu(gate) * up`` of a fused [rows, 2 f] activation."""
    rows, two_f = gate_up.shape
    out = torch.empty((rows, two_f // 2), device=gate_up.device, dtype=gate_up.dtype)
    if out.numel():
        gu = gate_up.contiguous()
        with _on_device(gu):
            st = nat.load().fxpr_silu_mul(gu.data_ptr(), nat.DTYPE_CODE[gu.dtype], out.data_ptr(), rows,
                                          two_f // 2, nat.stream_ptr(gu.device))
        nat.check(st, "silu_mul")
    return out


# --------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------

_gemm_scratch: dict[tuple[int, int], torch.Tensor] = {}
_gemm_scratch_retired: list[torch.Tensor] = []


def _get_gemm_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """Persistent zero-initialised split-K scratch per device, grown on demand
    (the kernel re-zeroes what it used; gemm.py:86-107 of the reference keeps
    one such buffer too).  ``warmup_gemm`` sizes it before CUDA-graph capture.
    A buffer that was replaced stays alive, so graphs captured with it keep a
    valid, still-zeroed counter region; growing *during* capture would allocate
    and zero-fill inside the graph, so that is refused."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    cur = _gemm_scratch.get((idx, 0))
    if cur is None or cur.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                f"gemm_fxp: split-K scratch of {nbytes} bytes needed during CUDA-graph capture but only "
                f"{0 if cur is None else cur.numel()} are allocated; run the shape once (or warmup_gemm) "
                "before capturing")
        if cur is not None:
            _gemm_scratch_retired.append(cur)
        cur = torch.zeros(max(nbytes, 1 << 20), device=device, dtype=torch.uint8)
        _gemm_scratch[(idx, 0)] = cur
    return cur


def gemm_scratch_policy_bytes(num_sms: int, int_bits: int = 64) -> int:
    """Largest scratch the automatic split-K policy (``pick_split_k``) can ask for,
    whatever M, N and K: it doubles the split only while ``tiles * split * 2 <= num_sms``,
    so at most ``num_sms`` integer partial tiles of 128 x 128 exist, each padded to 256
    columns in the worst case, after the fixed 256 KiB counter region."""
    planes = num_sms * 128 * 256 * (8 if int_bits == 64 else 4)
    return 256 * 1024 + -(-planes // 256) * 256


_status_words: dict[int, torch.Tensor] = {}


def _status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 the kernels set when a bounded device-side wait gives up."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(1, device=device, dtype=torch.int32)
        _status_words[idx] = t
    return t


def check_device_status(device=None) -> None:
    """Synchronise and raise if any kernel reported a timed-out wait since the
    last check (not on the hot path: tests, benchmarks and debugging call it)."""
    for idx, t in list(_status_words.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        v = int(t.item())
        if v != 0:
            t.zero_()
            nat.check(v, f"device status word on cuda:{idx}")


_SM_COUNT: dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _SM_COUNT.get(idx)
    if n is None:
        n = torch.cuda.get_device_properties(idx).multi_processor_count
        _SM_COUNT[idx] = n
    return n


def pick_split_k(M: int, N: int, K: int, k_tile: int, int_bits: int, num_sms: int) -> int:
    """Host-shape-only split-K policy (both routes give the same bits, so this
    is a speed decision only; the reference times it at warmup instead,
    gemm.py:780-836).  Split when the output tiles alone cannot fill the GPU."""
    if int_bits == 16:
        return 1
    tiles_mn = -(-M // 128) * -(-N // 128)
    k_tiles = -(-K // k_tile)
    if tiles_mn >= num_sms or k_tiles < 8:
        return 1
    if M <= 64:
        # decode shapes (cluster merge): the largest power of two that fills the SMs once --
        # clusters of CTAs that each take a whole SM do not pack the last tenth of the SMs --
        # and leaves every rank at least 384 of K (below that the fixed cost of a rank wins)
        split = 1
        while split < 8 and tiles_mn * split * 2 <= num_sms * 9 // 10 and K // (split * 2) >= 384:
            split *= 2
        return split
    split = 1
    # one wave of CTAs at most: a second, partly filled wave costs more than it hides
    while split < 16 and tiles_mn * split * 2 <= num_sms and k_tiles // (split * 2) >= 4:
        split *= 2
    return split


def _gemm_common(a, b, bias, int_bits, frac_bits, want_c: bool, want_int: bool, out_int=None,
                 silu_pairs: bool = False):
    M, K = a.shape
    N = b.shape[1]
    c = torch.empty((M, N // 2 if silu_pairs else N), device=a.device, dtype=a.dtype) if want_c else None
    if out_int is not None:
        if (out_int.shape != (M, N) or out_int.dtype != _INT_DTYPE[int_bits] or not out_int.is_contiguous()
                or out_int.device != a.device):
            raise ValueError("gemm_fxp_int_into: out must be a contiguous [M, N] tensor of the accumulator type")
        c_int = out_int
    else:
        c_int = torch.empty((M, N), device=a.device, dtype=_INT_DTYPE[int_bits]) if want_int else None
    if M == 0 or N == 0:
        return c, c_int
    if a.dtype not in _IO_DTYPES or b.dtype != a.dtype:
        raise TypeError(f"gemm_fxp: unsupported dtypes {a.dtype} x {b.dtype}")
    cfg = get_runtime_config()
    k_tile = _ovr.gemm_k_tile if _ovr.gemm_k_tile is not None else cfg.gemm_k_tile
    if not k_tile:
        k_tile = BLOCK_K_BY_DTYPE[a.dtype]
    split_k = _ovr.gemm_split_k if _ovr.gemm_split_k is not None else cfg.gemm_split_k
    if not split_k:
        split_k = pick_split_k(M, N, K, k_tile, int_bits, _sm_count(a.device))
    split_k = max(1, min(split_k, -(-K // k_tile) if K else 1))
    flags = (nat.GEMM_FORCE_PORTABLE if _ovr.gemm_portable else 0) | int(_ovr.gemm_flags)
    if silu_pairs:
        flags |= nat.GEMM_SILU_MUL
    lib = nat.load()
    scratch = None
    scratch_bytes = 0
    partials = None
    if _ovr.gemm_partials and split_k == 1:
        partials = torch.zeros((-(-K // k_tile) if K else 0, M, N), device=a.device,
                               dtype=torch.float32)
        _ovr.last_partials = partials
    if split_k > 1:
        scratch_bytes = lib.fxpr_gemm_scratch_bytes(M, N, int_bits, split_k)
        scratch = _get_gemm_scratch(a.device, scratch_bytes)
    if bias is not None and bias.dtype != a.dtype:
        bias = bias.to(a.dtype)
    with _on_device(a):
        st = lib.fxpr_gemm(
            a.data_ptr(), b.data_ptr(), nat.ptr(bias), nat.ptr(c), nat.ptr(c_int),
            nat.DTYPE_CODE[a.dtype], M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1),
            c.stride(0) if c is not None else N, int_bits, frac_bits, k_tile, split_k, flags,
            nat.ptr(scratch), scratch_bytes, nat.ptr(partials if partials is not None and partials.numel() else None),
            _status_word(a.device).data_ptr(), nat.stream_ptr(a.device))
    if silu_pairs and st == nat.FXPR_ERR_UNSUPPORTED:
        return None, None                       # the caller runs the two-kernel form
    nat.check(st, "gemm_fxp")
    return c, c_int


def gemm_fxp_run(a, b, bias, int_bits, fxp_frac_bits):
    """gemm.py:612-763 of the reference (no autotune: the kernels are AOT)."""
    c, _ = _gemm_common(a, b, bias, int_bits, fxp_frac_bits, True, False)
    return c


def gemm_fxp_int_run(a, b, int_bits, fxp_frac_bits):
    _, c_int = _gemm_common(a, b, None, int_bits, fxp_frac_bits, False, True)
    return c_int


def silu_mul_pairs(gate_up):
    """``silu(gate_up[:, 0::2]) * gate_up[:, 1::2]`` for an activation whose columns are
    (gate_j, up_j) pairs (the layout ``gemm_silu_mul`` keeps its weights in)."""
    if gate_up.dtype not in _IO_DTYPES or gate_up.dim() != 2 or gate_up.shape[1] % 2:
        raise TypeError("silu_mul_pairs: [rows, 2f] tensor of an io dtype expected")
    gate_up = gate_up.contiguous()
    rows, f = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, f), device=gate_up.device, dtype=gate_up.dtype)
    if rows and f:
        with _on_device(gate_up):
            st = nat.load().fxpr_silu_mul_pairs(gate_up.data_ptr(), nat.DTYPE_CODE[gate_up.dtype],
                                                out.data_ptr(), rows, f, nat.stream_ptr(gate_up.device))
        nat.check(st, "silu_mul_pairs")
    return out


def interleave_gate_up(w_gate, w_up):
    """``(K, f)`` gate and up weights -> ``(K, 2f)`` with columns (gate_0, up_0, gate_1, ...)."""
    return torch.stack([w_gate, w_up], dim=2).reshape(w_gate.shape[0], -1).contiguous()


def gemm_silu_mul(a, b_pairs, int_bits, fxp_frac_bits):
    """``silu(a @ gate) * (a @ up)`` with the gate and up columns of ``b_pairs`` interleaved
    (``interleave_gate_up``).  For at most 64 rows the decode-shape GEMM combines the column pairs
    in its epilogue; otherwise the GEMM and ``silu_mul_pairs`` run one after the other.  Same bits
    either way (and as ``gemm_fxp`` + ``silu_mul`` on the plain layout)."""
    if b_pairs.shape[1] % 2:
        raise ValueError("gemm_silu_mul: the weight needs an even number of columns")
    if a.shape[0] <= 64:
        c, _ = _gemm_common(a, b_pairs, None, int_bits, fxp_frac_bits, True, False, silu_pairs=True)
        if c is not None:
            return c
    return silu_mul_pairs(gemm_fxp_run(a, b_pairs, None, int_bits, fxp_frac_bits))


def gemm_fxp_argmax(a, b, bias, int_bits, fxp_frac_bits, n_offset: int = 0):
    """``gemm_fxp`` for at most 64 rows that also returns, per row, the arg-max key of the
    outputs (``int64 [M]``, see ``argmax_from_keys``): greedy sampling straight from the lm_head
    GEMM, with no pass over the ``[M, vocab]`` logits.  Keys of vocab shards (``n_offset`` = first
    column of the shard) combine with ``combine_argmax_keys``.  Shapes the fused kernel does not
    take fall back to ``gemm_fxp`` + a key built from ``torch.max``: same result."""
    M, K = a.shape
    N = b.shape[1]
    c = torch.empty((M, N), device=a.device, dtype=a.dtype)
    keys = torch.zeros((M,), device=a.device, dtype=torch.int64)
    if M == 0 or N == 0:
        return c, keys
    cfg = get_runtime_config()
    k_tile = _ovr.gemm_k_tile if _ovr.gemm_k_tile is not None else cfg.gemm_k_tile
    if not k_tile:
        k_tile = BLOCK_K_BY_DTYPE[a.dtype]
    flags = (nat.GEMM_FORCE_PORTABLE if _ovr.gemm_portable else 0) | int(_ovr.gemm_flags)
    st = nat.FXPR_ERR_UNSUPPORTED
    if M <= 64 and a.dtype in (torch.float16, torch.bfloat16) and b.dtype == a.dtype:
        if bias is not None and bias.dtype != a.dtype:
            bias = bias.to(a.dtype)
        with _on_device(a):
            st = nat.load().fxpr_gemm_argmax(
                a.data_ptr(), b.data_ptr(), nat.ptr(bias), c.data_ptr(), keys.data_ptr(), int(n_offset),
                nat.DTYPE_CODE[a.dtype], M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1),
                c.stride(0), int_bits, fxp_frac_bits, k_tile, flags, _status_word(a.device).data_ptr(),
                nat.stream_ptr(a.device))
    if st == nat.FXPR_ERR_UNSUPPORTED:
        c = gemm_fxp_run(a, b, bias, int_bits, fxp_frac_bits)
        return c, argmax_keys_of(c, n_offset)
    nat.check(st, "gemm_fxp_argmax")
    return c, keys


def argmax_keys_of(logits, n_offset: int = 0):
    """The key ``fxpr_gemm_argmax`` leaves for each row of ``logits`` (16-bit io dtypes)."""
    v, idx = logits.max(dim=-1)                     # first maximal column, as torch.argmax
    bits = v.float().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    ordv = torch.where(bits >= 0x80000000, (~bits) & 0xFFFFFFFF, bits | 0x80000000)
    return ((ordv << 32) | (0xFFFFFFFF - (idx.to(torch.int64) + int(n_offset)))) ^ torch.iinfo(torch.int64).min ^ torch.iinfo(torch.int64).min


def combine_argmax_keys(keys_list):
    """Keys of several vocab shards -> keys of the whole row (unsigned 64-bit maximum)."""
    flip = torch.iinfo(torch.int64).min
    stacked = torch.stack([k ^ flip for k in keys_list], dim=0)     # signed order == unsigned order
    return stacked.max(dim=0).values ^ flip


def argmax_from_keys(keys):
    """Winning column per row: the largest output, the smallest column among equals."""
    return 0xFFFFFFFF - (keys & 0xFFFFFFFF)


def gemm_fxp_int_into(a, b, out, int_bits, fxp_frac_bits):
    """``gemm_fxp_int`` into a caller-owned accumulator tensor (for example a peer-mapped
    buffer that other ranks read)."""
    _gemm_common(a, b, None, int_bits, fxp_frac_bits, False, True, out_int=out)
    return out


def gemm_fxp_epilogue_run(c_int, bias, out_dtype, fxp_frac_bits):
    if c_int.dtype not in _INT_BITS:
        raise TypeError(f"gemm_fxp_epilogue: c_int must be an integer tensor, got {c_int.dtype}")
    if out_dtype not in _IO_DTYPES:
        raise TypeError(f"gemm_fxp_epilogue: unsupported output dtype {out_dtype}")
    c_int = c_int.contiguous()
    M, N = c_int.shape
    c = torch.empty((M, N), device=c_int.device, dtype=out_dtype)
    if M == 0 or N == 0:
        return c
    if bias is not None and bias.dtype != out_dtype:
        bias = bias.to(out_dtype)
    with _on_device(c_int):
        st = nat.load().fxpr_gemm_epilogue_from_int(
            c_int.data_ptr(), _INT_BITS[c_int.dtype], nat.ptr(bias), c.data_ptr(),
            nat.DTYPE_CODE[out_dtype], M, N, c.stride(0), fxp_frac_bits,
            nat.stream_ptr(c_int.device))
    nat.check(st, "gemm_fxp_epilogue")
    return c


# --------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------

_MIN_KV_TILES_FOR_SPLIT = 32   # attention.py:46-48 of the reference
_MAX_NUM_SPLITS = 8
_SPLIT_BASE_OVERSUB = 2


def _next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def pick_num_splits(requested, num_requests, num_q_blocks, num_heads, num_kv_tiles, num_sms):
    """attention.py:664-689 of the reference: an explicit request wins; otherwise
    split only long contexts on an under-filled GPU, power of two, at most 8."""
    if requested >= 1:
        return requested
    if num_kv_tiles <= _MIN_KV_TILES_FOR_SPLIT:
        return 1
    base = max(1, num_requests * num_q_blocks * num_heads)
    if base > _SPLIT_BASE_OVERSUB * num_sms:
        return 1
    split = min(num_kv_tiles // _MIN_KV_TILES_FOR_SPLIT, _MAX_NUM_SPLITS)
    return _next_pow2(split) if split >= 2 else 1


def _tensor_core_route(q, kv_cache, num_heads, num_kv_heads, head_dim, page_size) -> bool:
    """Mirror of the C side's routing rule (dtype / geometry only, never batch)."""
    g = num_heads // num_kv_heads
    if not (q.dtype in (torch.float16, torch.bfloat16) and head_dim in (64, 128)
            and page_size % 16 == 0 and g in (1, 2, 4, 8, 16) and not _ovr.attn_portable):
        return False
    # 16-byte copies: row starts must be 16-byte aligned
    strides = (q.stride(0), q.stride(1), kv_cache.stride(0), kv_cache.stride(2), kv_cache.stride(3))
    if any(st % 8 for st in strides):
        return False
    return (q.data_ptr() | kv_cache.data_ptr() | kv_cache.select(1, 1).data_ptr()) % 16 == 0


def pick_num_splits_b200(requested, num_requests, max_query_len, num_heads, num_kv_heads,
                         max_keys, num_sms):
    """Split policy of the tensor-core route, where splits are cluster ranks: results do
    not depend on it, so it only balances the GPU.  Decode keeps each CTA's key slice near
    1024 keys (small score stash -> more resident CTAs) unless fewer clusters than CTA slots call for more ranks; prefill splits only when the row
    blocks alone cannot fill the SMs.  Host shapes only, so it is fixed under a CUDA graph."""
    if requested >= 1:
        return min(requested, 16)
    g = num_heads // num_kv_heads
    if max_query_len * g <= 16:
        # A rank's score stash must leave room for four CTAs per SM (about 19.5 KB: 19 key tiles
        # at 16 bytes per key), which sets the least rank count for long contexts.  Few clusters:
        # enough ranks to fill one wave of 4 CTAs per SM, at least two key tiles each.  Measured
        # on 64 requests x 1152 keys: 8 KV heads 70 -> 63 us with 1 rank instead of 2 (when the
        # block table is no wider than that), 2 KV heads 30 -> 20.5 us with 4, 1 KV head 25 -> 16 us
        # with 8.
        tiles = -(-max_keys // 64)
        key_bytes = 4 * g if g <= 8 else 64
        budget = 19968 + (2048 if g <= 8 else 0)      # eight-row Q tiles leave 2 KB more
        cap_tiles = max(1, (budget // key_bytes) // 64)
        by_keys = -(-tiles // cap_tiles)
        by_keys = 8 if by_keys > 4 else max(1, by_keys)
        clusters = max(1, num_requests * num_kv_heads)
        by_fill = max(1, min(8, (4 * num_sms) // clusters, tiles // 2))
        return max(by_keys, by_fill)
    rows_per_block = 64
    blocks = num_requests * num_kv_heads * max(1, -(-(max_query_len * g) // rows_per_block))
    if blocks >= num_sms or max_keys <= 2048:
        return 1
    return max(1, min(8, num_sms // blocks))


def unified_attention_fxp_run(q, kv_cache, o, query_start_loc, seq_lens, block_table,
                              max_query_len, alibi_slopes, is_causal, softmax_scale,
                              fxp_int_bits, fxp_frac_bits, logit_softcap, window_size,
                              num_kv_splits):
    """attention.py:692-953 of the reference: same validation, same split policy."""
    if not (q.is_cuda and kv_cache.is_cuda and o.is_cuda):
        raise RuntimeError("unified_attention_fxp: tensors must be CUDA")
    if q.dtype not in _IO_DTYPES:
        raise TypeError(f"unified_attention_fxp: unsupported q dtype {q.dtype}")
    if kv_cache.dim() != 5 or kv_cache.shape[1] != 2:
        raise ValueError("kv_cache must be (num_blocks, 2, page_size, num_kv_heads, head_dim)")
    if kv_cache.dtype != q.dtype or o.dtype != q.dtype:
        raise TypeError("kv_cache and o must share dtype with q")
    if query_start_loc.dtype != torch.int32:
        raise TypeError("query_start_loc must be int32")
    if seq_lens.dtype != torch.int32:
        raise TypeError("seq_lens must be int32")
    if block_table.dtype != torch.int32:
        raise TypeError("block_table must be int32")
    if num_kv_splits < 0:
        raise ValueError(f"num_kv_splits must be >= 0, got {num_kv_splits}")
    has_alibi = alibi_slopes is not None and alibi_slopes.numel() > 0
    if has_alibi and alibi_slopes.dtype != torch.float32:
        raise TypeError("alibi_slopes must be float32")

    num_heads, head_dim = q.shape[1], q.shape[2]
    page_size, num_kv_heads = kv_cache.shape[2], kv_cache.shape[3]
    num_requests = seq_lens.shape[0]
    if num_heads % num_kv_heads != 0:
        raise ValueError("num_heads must be divisible by num_kv_heads")
    if num_requests == 0 or q.shape[0] == 0:
        return
    if q.stride(2) != 1 or o.stride(2) != 1 or kv_cache.stride(4) != 1:
        raise ValueError("unified_attention_fxp: head_dim must be the unit-stride dimension")

    ss = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(head_dim)
    block_m = 16 if max_query_len <= 1 else 32
    block_n = BLOCK_N_BY_DTYPE[q.dtype]
    num_q_blocks = max(1, -(-max(1, int(max_query_len)) // block_m))
    max_kv_blocks = block_table.shape[1] if block_table.dim() == 2 else 0
    num_kv_tiles = -(-max(1, max_kv_blocks * page_size) // block_n)
    tensor_core = _tensor_core_route(q, kv_cache, num_heads, num_kv_heads, head_dim, page_size)
    if tensor_core:
        splits = pick_num_splits_b200(int(num_kv_splits), num_requests, int(max_query_len),
                                      num_heads, num_kv_heads, max(1, max_kv_blocks * page_size),
                                      _sm_count(q.device))
    else:
        splits = pick_num_splits(int(num_kv_splits), num_requests, num_q_blocks, num_heads,
                                 num_kv_tiles, _sm_count(q.device))

    lib = nat.load()
    scratch = None
    scratch_bytes = 0
    if splits > 1 and not tensor_core:
        # only the CUDA-core route keeps per-split maxima, integer totals and arrival counters
        # in scratch; the tensor-core kernels merge their splits inside a thread-block cluster
        scratch_bytes = lib.fxpr_attention_scratch_bytes(q.shape[0], num_heads, head_dim,
                                                         fxp_int_bits, splits)
        scratch = torch.empty(scratch_bytes, device=q.device, dtype=torch.uint8)
    alibi = alibi_slopes.contiguous() if has_alibi else None
    flags = ((nat.ATTN_CAUSAL if is_causal else 0) | (nat.ATTN_FORCE_PORTABLE if _ovr.attn_portable else 0)
             | int(_ovr.attn_flags))
    k_cache = kv_cache.select(1, 0)
    v_cache = kv_cache.select(1, 1)
    qsl = query_start_loc.contiguous()
    sl = seq_lens.contiguous()
    bt_stride = block_table.stride(0) if block_table.dim() == 2 else 0
    if block_table.dim() == 2 and block_table.stride(1) != 1:
        block_table = block_table.contiguous()
        bt_stride = block_table.stride(0)
    with _on_device(q):
        st = lib.fxpr_attention(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), o.data_ptr(),
            qsl.data_ptr(), sl.data_ptr(), block_table.data_ptr(), nat.ptr(alibi),
            nat.DTYPE_CODE[q.dtype], q.shape[0], num_requests, num_heads, num_kv_heads,
            head_dim, page_size, q.stride(0), q.stride(1), o.stride(0), o.stride(1),
            kv_cache.stride(0), kv_cache.stride(2), kv_cache.stride(3), bt_stride,
            int(max_query_len), flags, ss, float(logit_softcap), int(window_size),
            fxp_int_bits, fxp_frac_bits, splits, nat.ptr(scratch), scratch_bytes,
            _status_word(q.device).data_ptr(),
            nat.stream_ptr(q.device))
    nat.check(st, "unified_attention_fxp")


# --------------------------------------------------------------------------
# dispatcher registrations (CUDA key only)
# --------------------------------------------------------------------------

@torch.library.impl("fxpr::float_to_fixed", "CUDA", lib=_lib)
def _float_to_fixed_cuda(x, int_bits, fxp_frac_bits):
    _check_int_bits(int_bits)
    _check_frac_bits(fxp_frac_bits)
    return float_to_fixed_run(x, int(int_bits), int(fxp_frac_bits))


@torch.library.impl("fxpr::fixed_to_float", "CUDA", lib=_lib)
def _fixed_to_float_cuda(x, float_bits, fxp_frac_bits):
    if int(float_bits) not in (16, 32, 64):
        raise ValueError(f"float_bits must be 16/32/64, got {float_bits}")
    _check_frac_bits(fxp_frac_bits)
    return fixed_to_float_run(x, int(float_bits), int(fxp_frac_bits))


@torch.library.impl("fxpr::rms_norm_fxp", "CUDA", lib=_lib)
def _rms_norm_fxp_cuda(x, weight, eps):
    return rms_norm_fxp_run(x, weight, float(eps))


@torch.library.impl("fxpr::rms_norm_fxp_from_int", "CUDA", lib=_lib)
def _rms_norm_fxp_from_int_cuda(acc, residual, weight, bias, eps, gemm_frac_bits):
    return rms_norm_fxp_from_int_run(acc, residual, weight, bias, float(eps), int(gemm_frac_bits))


@torch.library.impl("fxpr::rms_norm_fxp_residual", "CUDA", lib=_lib)
def _rms_norm_fxp_residual_cuda(x, residual, weight, eps):
    return rms_norm_fxp_residual_run(x, residual, weight, float(eps))


@torch.library.impl("fxpr::gemm_fxp", "CUDA", lib=_lib)
def _gemm_fxp_cuda(a, b, bias, fxp_int_bits, fxp_frac_bits):
    _check_int_bits(fxp_int_bits)
    _check_frac_bits(fxp_frac_bits)
    return gemm_fxp_run(a, b, bias, int(fxp_int_bits), int(fxp_frac_bits))


@torch.library.impl("fxpr::unified_attention_fxp", "CUDA", lib=_lib)
def _unified_attention_fxp_cuda(q, kv_cache, o, query_start_loc, seq_lens, block_table,
                                max_query_len, alibi_slopes, is_causal, softmax_scale,
                                fxp_int_bits, fxp_frac_bits, logit_softcap, window_size,
                                num_kv_splits):
    _check_int_bits(fxp_int_bits)
    _check_frac_bits(fxp_frac_bits)
    unified_attention_fxp_run(
        q, kv_cache, o, query_start_loc, seq_lens, block_table, int(max_query_len),
        alibi_slopes, bool(is_causal),
        None if softmax_scale is None else float(softmax_scale),
        int(fxp_int_bits), int(fxp_frac_bits), float(logit_softcap), int(window_size),
        int(num_kv_splits))


@torch.library.impl("fxpr::log_softmax_fxp", "CUDA", lib=_lib)
def _log_softmax_fxp_cuda(x, fxp_frac_bits):
    _check_frac_bits(fxp_frac_bits)
    return log_softmax_fxp_run(x, int(fxp_frac_bits))


@torch.library.impl("fxpr::gemm_fxp_int", "CUDA", lib=_lib)
def _gemm_fxp_int_cuda(a, b, fxp_int_bits, fxp_frac_bits):
    _check_int_bits(fxp_int_bits)
    _check_frac_bits(fxp_frac_bits)
    return gemm_fxp_int_run(a, b, int(fxp_int_bits), int(fxp_frac_bits))


@torch.library.impl("fxpr::gemm_fxp_epilogue", "CUDA", lib=_lib)
def _gemm_fxp_epilogue_cuda(c_int, bias, out_dtype, fxp_frac_bits):
    _check_frac_bits(fxp_frac_bits)
    return gemm_fxp_epilogue_run(c_int, bias, out_dtype, int(fxp_frac_bits))
