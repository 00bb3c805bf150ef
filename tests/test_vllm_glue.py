"""The vLLM-facing glue: plugin entry point, ``register()``, the ``fixedpoint``
quantization methods, the ``CUSTOM`` attention backend, ``DeterministicRMSNorm``
and the sampler hook (``fxpr_vllm/register.py``, ``monkey_patches.py``,
``quantisation_config.py``, ``attention_backend.py``, ``rms_norm.py`` of the
reference, plus the sampler the reference's README names but does not ship).

CPU tests check what registration does to vLLM's registries (in a child process,
because it replaces classes process-wide) and the host logic of the methods on
stub layers; GPU tests drive ``forward`` / ``apply`` on stub layers and compare
with the operators called directly.
"""
from __future__ import annotations

import json
import subprocess
import sys
import tomllib
import types
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "vllm-triton-fixed-point-reductions_b200"

vllm = pytest.importorskip("vllm")

_REGISTER_PROBE = r"""
import json, sys
sys.path.insert(0, %(pkg)r)
import torch
import fxpr_vllm
from fxpr_vllm.register import register
register()
register()      # idempotent: a second call must change nothing and not raise
from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS, get_quantization_config
from vllm.v1.attention.backends.registry import AttentionBackendEnum
from vllm.model_executor.custom_op import op_registry, op_registry_oot
import vllm.model_executor.layers.layernorm as layernorm_mod
from vllm.v1.sample.sampler import Sampler
cfg = get_quantization_config("fixedpoint")
lp = Sampler.compute_logprobs(torch.randn(3, 11))
out = {
    "quant_listed": "fixedpoint" in QUANTIZATION_METHODS,
    "quant_cls": cfg.__module__ + "." + cfg.__qualname__,
    "quant_name": cfg.get_name(),
    "backend_path": AttentionBackendEnum.CUSTOM.get_path(),
    "backend_name": AttentionBackendEnum.CUSTOM.get_class().get_name(),
    "rms_op": op_registry["rms_norm"].__qualname__,
    "rms_oot": op_registry_oot["RMSNorm"].__qualname__ if "RMSNorm" in op_registry_oot else None,
    "rms_mod": layernorm_mod.RMSNorm.__qualname__,
    "sampler_patched": bool(getattr(Sampler.compute_logprobs, "_fxpr_patched", False)),
    "sampler_cpu_rows_sum_to_one": bool(torch.allclose(lp.exp().sum(-1), torch.ones(3), atol=1e-5)),
}
print("PROBE" + json.dumps(out))
"""


def _run_probe(env_extra=None):
    import os

    env = dict(os.environ)
    env.update(env_extra or {})
    r = subprocess.run([sys.executable, "-c", _REGISTER_PROBE % {"pkg": str(PKG)}], capture_output=True,
                       text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("PROBE")][-1]
    return json.loads(line[5:])


def test_register_installs_every_surface_and_is_idempotent():
    got = _run_probe()
    assert got["quant_listed"] and got["quant_name"] == "fixedpoint"
    assert got["quant_cls"] == "fxpr_vllm.quantisation_config.FixedPointConfig"
    assert got["backend_path"] == "fxpr_vllm.attention_backend.DeterministicAttentionBackend"
    assert got["backend_name"] == "CUSTOM"
    assert got["rms_op"] == got["rms_oot"] == got["rms_mod"] == "DeterministicRMSNorm"
    assert got["sampler_patched"] and got["sampler_cpu_rows_sum_to_one"]


def test_disable_switches_leave_vllm_classes_alone():
    got = _run_probe({"FXPR_DISABLE_RMS_NORM": "1", "FXPR_DISABLE_SAMPLER": "1"})
    assert got["quant_listed"] and got["backend_name"] == "CUSTOM"
    assert got["rms_mod"] == "RMSNorm" and got["rms_op"] == "RMSNorm" and got["rms_oot"] is None
    assert not got["sampler_patched"]


def test_pyproject_declares_the_reference_entry_point():
    meta = tomllib.loads((PKG / "pyproject.toml").read_text())
    eps = meta["project"]["entry-points"]["vllm.general_plugins"]
    assert eps == {"fxpr_vllm": "fxpr_vllm.register:register"}   # reference pyproject.toml:12-13
    mod_name, fn_name = eps["fxpr_vllm"].split(":")
    import importlib

    assert callable(getattr(importlib.import_module(mod_name), fn_name))
    assert meta["project"]["name"] == "fxpr_vllm"


def test_warm_scratch_is_bounded_by_the_split_policy_not_by_n():
    from fxpr_vllm import _lib as L

    # lm_head-sized N must not pin gigabytes at load time
    assert L.gemm_scratch_policy_bytes(148, 64) <= 64 << 20
    # and the bound really covers what the policy can ask for
    lib = __import__("fxpr_vllm._native", fromlist=["load"]).load()
    for (m, n, k) in [(64, 4096, 4096), (64, 128256, 4096), (64, 4096, 14336), (256, 6144, 4096),
                      (1, 28672, 4096), (512, 1024, 8192), (130, 384, 16384)]:
        for kt in (64, 128):
            s = L.pick_split_k(m, n, k, kt, 64, 148)
            if s > 1:
                assert lib.fxpr_gemm_scratch_bytes(m, n, 64, s) <= L.gemm_scratch_policy_bytes(148, 64), (m, n, k, s)


class _StubRowParallel:
    """Set up below as an instance of vLLM's RowParallelLinear without running its
    constructor (which needs an initialised TP group)."""


def _stub_row_parallel(k_shard, n, tp, dtype=torch.bfloat16, input_size=None):
    from vllm.model_executor.layers.linear import RowParallelLinear

    layer = RowParallelLinear.__new__(RowParallelLinear)
    torch.nn.Module.__init__(layer)
    layer.tp_size = tp
    layer.reduce_results = True
    layer.skip_bias_add = False
    layer.input_size = input_size if input_size is not None else k_shard * tp
    layer.weight_native = torch.zeros(k_shard, n, dtype=dtype)
    return layer


def test_setup_tp_checks_that_the_shards_are_whole_k_tiles():
    from fxpr_vllm.quantisation_config import FixedPointConfig, FixedPointLinearMethod

    m = FixedPointLinearMethod(FixedPointConfig())
    good = _stub_row_parallel(1024, 64, 4)          # 4096 / 4 = 8 K-tiles of 128 per rank
    m._setup_tp(good)
    assert good._fxp_int_reduce is True and good.reduce_results is False
    bad = _stub_row_parallel(192, 64, 2)            # 192 is not a whole number of 128-deep tiles
    m._setup_tp(bad)
    assert bad._fxp_int_reduce is False and bad.reduce_results is True   # vLLM's reduce stays on
    single = _stub_row_parallel(4096, 64, 1)
    m._setup_tp(single)
    assert single._fxp_int_reduce is False and single.reduce_results is True


def test_quant_config_surface():
    from vllm.model_executor.layers.linear import LinearBase

    from fxpr_vllm.quantisation_config import (FixedPointConfig, FixedPointEmbeddingMethod,
                                               FixedPointLinearMethod)

    cfg = FixedPointConfig.from_config({})
    assert cfg.get_name() == "fixedpoint"
    assert torch.bfloat16 in cfg.get_supported_act_dtypes() and cfg.get_config_filenames() == []
    lin = LinearBase.__new__(LinearBase)
    assert isinstance(cfg.get_quant_method(lin, "x"), FixedPointLinearMethod)
    assert cfg.get_quant_method(torch.nn.ReLU(), "x") is None
    m = FixedPointEmbeddingMethod(cfg)
    layer = torch.nn.Module()
    m.create_weights(layer, 8, [5, 3], 8, 8, torch.float32)
    assert layer.weight.shape == (8, 8)
    layer.weight.data.copy_(torch.arange(64.0).reshape(8, 8))   # create_weights leaves it uninitialised (may hold NaN)
    idx = torch.tensor([1, 7])
    assert torch.equal(m.embedding(layer, idx), layer.weight[idx])


def test_backend_class_contract():
    from fxpr_vllm.attention_backend import DeterministicAttentionBackend as B
    from fxpr_vllm.attention_backend import DeterministicAttentionImpl

    assert B.get_name() == "CUSTOM"
    assert B.get_kv_cache_shape(7, 32, 8, 128) == (7, 2, 32, 8, 128)
    with pytest.raises(ValueError):
        B.get_kv_cache_shape(7, 24, 8, 128)
    assert B.supports_head_size(32) and not B.supports_head_size(16)
    assert B.get_impl_cls() is DeterministicAttentionImpl
    with pytest.raises(NotImplementedError):
        DeterministicAttentionImpl(8, 64, 0.125, 2, None, None, kv_cache_dtype="fp8")
    impl = DeterministicAttentionImpl(4, 64, 0.125, 2, [0.5, 0.25, 0.125, 0.0625], 128, logits_soft_cap=30.0)
    assert torch.allclose(impl.alibi_slopes, torch.tensor([0.5, 0.25, 0.125, 0.0625]) * 1.4426950408889634)
    assert impl.window_size == 128 and impl.logits_soft_cap == 30.0


# ----------------------------------------------------------------------------------
# GPU: the glue classes against the operators called directly
# ----------------------------------------------------------------------------------

@pytest.mark.gpu
def test_attention_impl_forward_equals_the_op_and_copies_back_other_dtypes():
    import fxpr_vllm  # noqa: F401
    from fxpr_vllm import synthetic as syn
    from fxpr_vllm.attention_backend import DeterministicAttentionImpl
    from fxpr_vllm.config import get_runtime_config

    rt = get_runtime_config()
    hq, hkv, d = 32, 8, 128
    lens, qlens = [300, 77, 1029], [1, 5, 1]
    q, kv, qsl, sl, bt = syn.paged_attention_inputs(lens, qlens, q_heads=hq, kv_heads=hkv, head_dim=d, seed=7)
    impl = DeterministicAttentionImpl(hq, d, d ** -0.5, hkv, None, None)
    meta = types.SimpleNamespace(query_start_loc=qsl, seq_lens=sl, block_table=bt, max_query_len=max(qlens))
    tokens = q.shape[0]

    expect = torch.empty_like(q)
    torch.ops.fxpr.unified_attention_fxp(q, kv, expect, qsl, sl, bt, max(qlens), None, True, d ** -0.5,
                                         rt.fxp_int_bits, rt.fxp_frac_bits, 0.0, 0, 0)
    out = torch.full((tokens, hq * d), float("nan"), device="cuda", dtype=q.dtype)
    got = impl.forward(None, q.view(tokens, hq * d), None, None, kv, meta, output=out)
    assert got.data_ptr() == out.data_ptr() and torch.equal(out.view_as(expect), expect)

    # a caller buffer of another dtype receives the converted result (the reference writes
    # it to a temporary and the caller never sees it: attention_backend.py:230-231, 251)
    out32 = torch.full((tokens, hq * d), float("nan"), device="cuda", dtype=torch.float32)
    impl.forward(None, q.view(tokens, hq * d), None, None, kv, meta, output=out32)
    assert torch.equal(out32.view_as(expect), expect.float())

    # a block table as wide as the model's maximum length (vLLM's): the backend hands the kernel
    # only the pages of the longest live sequence, and the bits stay the same
    wide = torch.zeros((bt.shape[0], 4 * bt.shape[1]), dtype=bt.dtype, device=bt.device)
    wide[:, : bt.shape[1]] = bt
    meta_w = types.SimpleNamespace(query_start_loc=qsl, seq_lens=sl, block_table=wide, max_query_len=max(qlens),
                                   max_seq_len=max(lens))
    out_w = torch.full((tokens, hq * d), float("nan"), device="cuda", dtype=q.dtype)
    impl.forward(None, q.view(tokens, hq * d), None, None, kv, meta_w, output=out_w)
    assert torch.equal(out_w.view_as(expect), expect)

    # the memory-profiling run (no metadata) returns zeros
    z = impl.forward(None, q.view(tokens, hq * d), None, None, kv, None)
    assert not z.any()


@pytest.mark.gpu
def test_linear_method_process_weights_and_apply_equal_the_gemm_op(monkeypatch):
    import fxpr_vllm  # noqa: F401
    import vllm.model_executor.parameter as vparam

    # vLLM's weight parameters ask the (uninitialised) TP group for rank and size
    monkeypatch.setattr(vparam, "get_tensor_model_parallel_rank", lambda: 0)
    monkeypatch.setattr(vparam, "get_tensor_model_parallel_world_size", lambda: 1)
    from fxpr_vllm.config import get_runtime_config
    from fxpr_vllm.quantisation_config import (FixedPointConfig, FixedPointEmbeddingMethod,
                                               FixedPointLinearMethod)

    rt = get_runtime_config()
    g = torch.Generator(device="cuda").manual_seed(11)
    n_out, k_in = 384, 512
    m = FixedPointLinearMethod(FixedPointConfig())
    layer = torch.nn.Module()
    m.create_weights(layer, k_in, [256, 128], k_in, n_out, torch.bfloat16, weight_loader=lambda *a, **k: None)
    assert layer.weight.shape == (n_out, k_in)
    layer.to("cuda")
    w = (0.05 * torch.randn(n_out, k_in, generator=g, device="cuda")).to(torch.bfloat16)
    layer.weight.data.copy_(w)
    m.process_weights_after_loading(layer)
    assert layer.weight is None and layer.weight_native.shape == (k_in, n_out)
    assert layer.weight_native.is_contiguous() and torch.equal(layer.weight_native, w.t())
    x = torch.randn(3, 5, k_in, generator=g, device="cuda").to(torch.bfloat16)
    bias = torch.randn(n_out, generator=g, device="cuda").to(torch.bfloat16)
    got = m.apply(layer, x.view(-1, k_in), bias)
    expect = torch.ops.fxpr.gemm_fxp(x.view(-1, k_in), w.t().contiguous(), bias, rt.fxp_int_bits, rt.fxp_frac_bits)
    assert torch.equal(got, expect)

    e = FixedPointEmbeddingMethod(FixedPointConfig())
    head = torch.nn.Module()
    e.create_weights(head, k_in, [n_out], k_in, n_out, torch.bfloat16)
    head.to("cuda")
    head.weight.data.copy_(w)
    e.process_weights_after_loading(head)
    assert torch.equal(e.apply(head, x.view(-1, k_in)),
                       torch.ops.fxpr.gemm_fxp(x.view(-1, k_in), w.t().contiguous(), None, rt.fxp_int_bits,
                                               rt.fxp_frac_bits))
    ids = torch.tensor([0, 5, 383], device="cuda")
    assert torch.equal(e.embedding(head, ids), w[ids])


@pytest.mark.gpu
def test_rms_norm_module_and_sampler_hook_equal_the_ops():
    import fxpr_vllm  # noqa: F401
    from fxpr_vllm import monkey_patches
    from fxpr_vllm.config import get_runtime_config
    from fxpr_vllm.rms_norm import DeterministicRMSNorm
    from vllm.v1.sample.sampler import Sampler

    g = torch.Generator(device="cuda").manual_seed(12)
    hidden = 1024
    norm = DeterministicRMSNorm.__new__(DeterministicRMSNorm)
    torch.nn.Module.__init__(norm)
    norm.variance_epsilon = 1e-6
    norm.weight = torch.nn.Parameter((1 + 0.1 * torch.randn(hidden, generator=g, device="cuda")).to(torch.bfloat16))
    x = torch.randn(9, hidden, generator=g, device="cuda").to(torch.bfloat16)
    r = torch.randn(9, hidden, generator=g, device="cuda").to(torch.bfloat16)
    assert torch.equal(norm.forward_cuda(x), torch.ops.fxpr.rms_norm_fxp(x, norm.weight, 1e-6))
    r1, r2 = r.clone(), r.clone()
    y, res = norm.forward_native(x, r1)
    assert res.data_ptr() == r1.data_ptr()
    assert torch.equal(y, torch.ops.fxpr.rms_norm_fxp_residual(x, r2, norm.weight, 1e-6)) and torch.equal(r1, r2)

    original = Sampler.__dict__["compute_logprobs"]
    try:
        monkey_patches.patch_sampler()
        logits = 2 * torch.randn(5, 32000, generator=g, device="cuda")
        got = Sampler.compute_logprobs(logits)
        assert torch.equal(got, torch.ops.fxpr.log_softmax_fxp(logits, get_runtime_config().fxp_frac_bits))
        assert got.dtype == torch.float32
        assert torch.allclose(got, logits.log_softmax(-1), atol=1e-4)
        monkey_patches.patch_sampler()          # idempotent
        assert Sampler.compute_logprobs._fxpr_original is original.__func__
    finally:
        Sampler.compute_logprobs = original
