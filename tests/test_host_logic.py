"""Host-side logic that needs no GPU: the C-ABI library loads and exports every
symbol the header declares, schemas/fakes match the reference's contract, env
knobs, split policies, and the constants shared by oracle and device code."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import fxpr_vllm  # noqa: F401
from fxpr_vllm import _lib as L
from fxpr_vllm import _native as nat
from fxpr_vllm import config as cfgmod
from oracle import fxp_oracle as orc

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "fxpr_b200.h"
CSRC = ROOT / "vllm-triton-fixed-point-reductions_b200" / "csrc"


def _declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(fxpr_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(nat.LIB_PATH))
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(nat.SIGNATURES) == names
    loaded = nat.load()
    assert loaded.fxpr_version() >= 100
    assert loaded.fxpr_status_string(-3).decode().startswith("scratch")


def test_argument_errors_without_a_gpu():
    lib = nat.load()
    # pure argument validation happens before any CUDA call
    assert lib.fxpr_float_to_fixed(None, nat.FXPR_F32, None, 24, 16, 4, None) == nat.FXPR_ERR_BAD_ARG
    assert lib.fxpr_float_to_fixed(None, nat.FXPR_F32, None, 32, 16, 0, None) == nat.FXPR_OK
    assert lib.fxpr_rms_norm(None, None, None, None, nat.FXPR_F32, 0, 64, 1e-6, 16, None) == nat.FXPR_OK
    assert lib.fxpr_gemm_scratch_bytes(64, 4096, 64, 1) == 0
    assert lib.fxpr_gemm_scratch_bytes(64, 4096, 64, 4) >= 64 * 4096 * 8
    assert lib.fxpr_attention_scratch_bytes(64, 32, 128, 64, 1) == 0
    assert lib.fxpr_attention_scratch_bytes(64, 32, 128, 64, 8) >= 64 * 32 * 128 * 8
    with pytest.raises(ValueError):
        nat.check(nat.FXPR_ERR_BAD_ARG, "x")
    with pytest.raises(TypeError):
        nat.check(nat.FXPR_ERR_UNSUPPORTED, "x")
    with pytest.raises(RuntimeError):
        nat.check(nat.FXPR_ERR_SCRATCH, "x")


def test_schemas_match_reference_strings():
    want = {
        "float_to_fixed": "fxpr::float_to_fixed(Tensor x, int int_bits, int fxp_frac_bits) -> Tensor",
        "fixed_to_float": "fxpr::fixed_to_float(Tensor x, int float_bits, int fxp_frac_bits) -> Tensor",
        "rms_norm_fxp": "fxpr::rms_norm_fxp(Tensor x, Tensor weight_fp32, float eps) -> Tensor",
        "rms_norm_fxp_residual": "fxpr::rms_norm_fxp_residual(Tensor x, Tensor(a!) residual, Tensor weight_fp32, float eps) -> Tensor",
        "gemm_fxp": "fxpr::gemm_fxp(Tensor a, Tensor b, Tensor? bias, int fxp_int_bits, int fxp_frac_bits) -> Tensor",
    }
    for name, schema in want.items():
        assert str(getattr(torch.ops.fxpr, name).default._schema) == schema
    s = str(torch.ops.fxpr.unified_attention_fxp.default._schema)
    assert "Tensor(a!) o" in s and s.endswith("int num_kv_splits) -> ()")


def test_cpu_tensors_are_rejected_not_emulated():
    x = torch.randn(4, 8)
    with pytest.raises(NotImplementedError):
        torch.ops.fxpr.float_to_fixed(x, 32, 16)
    with pytest.raises(NotImplementedError):
        torch.ops.fxpr.gemm_fxp(x, x.t().contiguous(), None, 32, 16)
    with pytest.raises(NotImplementedError):
        torch.ops.fxpr.rms_norm_fxp(x, torch.ones(8), 1e-6)


def test_fake_impls_shapes_and_dtypes():
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(3, 8, dtype=torch.float16)
        assert torch.ops.fxpr.float_to_fixed(x, 64, 16).dtype == torch.int64
        assert torch.ops.fxpr.fixed_to_float(x.to(torch.int32), 64, 16).dtype == torch.float64
        assert torch.ops.fxpr.rms_norm_fxp(x, torch.empty(8, dtype=torch.float16), 1e-6).shape == (3, 8)
        b = torch.empty(8, 5, dtype=torch.float16)
        out = torch.ops.fxpr.gemm_fxp(x, b, None, 32, 16)
        assert out.shape == (3, 5) and out.dtype == torch.float16
        assert torch.ops.fxpr.gemm_fxp_int(x, b, 64, 16).dtype == torch.int64
        assert torch.ops.fxpr.log_softmax_fxp(x, 16).dtype == torch.float32


def test_env_knobs(monkeypatch):
    for k in ("FXPR_INT_BITS", "FXPR_FRAC_BITS", "FXPR_DISABLE_RMS_NORM", "FXPR_GEMM_KTILE"):
        monkeypatch.delenv(k, raising=False)
    c = cfgmod.load_runtime_config()
    assert (c.fxp_int_bits, c.fxp_frac_bits, c.enable_rms_norm, c.enable_lm_head) == (32, 16, True, True)
    monkeypatch.setenv("FXPR_INT_BITS", "64")
    monkeypatch.setenv("FXPR_FRAC_BITS", "8")
    monkeypatch.setenv("FXPR_DISABLE_RMS_NORM", "1")
    monkeypatch.setenv("FXPR_GEMM_KTILE", "64")
    c = cfgmod.load_runtime_config()
    assert (c.fxp_int_bits, c.fxp_frac_bits, c.enable_rms_norm, c.gemm_k_tile) == (64, 8, False, 64)
    monkeypatch.setenv("FXPR_INT_BITS", "48")      # invalid -> default
    monkeypatch.setenv("FXPR_FRAC_BITS", "abc")    # malformed -> default
    c = cfgmod.load_runtime_config()
    assert (c.fxp_int_bits, c.fxp_frac_bits) == (32, 16)


def test_attention_split_policy_matches_reference_rules():
    # attention.py:664-689 of the reference
    assert L.pick_num_splits(5, 64, 1, 32, 1000, 148) == 5          # explicit wins
    assert L.pick_num_splits(0, 1, 1, 32, 32, 148) == 1             # short context
    assert L.pick_num_splits(0, 64, 1, 32, 128, 148) == 1           # GPU already full
    assert L.pick_num_splits(0, 1, 1, 32, 64, 148) == 2
    assert L.pick_num_splits(0, 1, 1, 32, 96, 148) == 4             # 3 -> next pow2
    assert L.pick_num_splits(0, 1, 1, 32, 4096, 148) == 8           # capped


def test_gemm_split_policy_is_bounded():
    for M, N, K in [(64, 4096, 4096), (1, 128256, 4096), (4096, 4096, 4096), (64, 4096, 14336)]:
        for kt in (64, 128):
            s = L.pick_split_k(M, N, K, kt, 64, 148)
            assert s in (1, 2, 4, 8, 16) and s <= max(1, K // kt)
    assert L.pick_split_k(4096, 4096, 4096, 64, 64, 148) == 1
    assert L.pick_split_k(64, 4096, 4096, 64, 16, 148) == 1         # no int16 atomics


def test_device_constants_equal_oracle_constants():
    text = (CSRC / "fxp_common.cuh").read_text()
    coefs = {int(k): int(v, 16) for v, k in re.findall(r"__int_as_float\((0x[0-9a-f]+)\)\S*\s*// c(\d)", text)}
    assert sorted(coefs) == list(range(8))
    for k, bits in coefs.items():
        assert np.float32(orc._EXP2_COEF[k]).view(np.uint32) == bits
    assert "0x3fb8aa3b" in text and np.float32(orc.RCP_LN2).view(np.uint32) == 0x3FB8AA3B
    for d in (19, 17, 15, 13, 11, 9, 7, 5, 3):
        assert (1.0 / d).hex().replace("0x1.", "0x1.") in text
    assert (orc._LN2_F64).hex() in text and (orc._SQRT_HALF_F64).hex() in text


def test_overrides_context_restores_state():
    with L.overrides(gemm_k_tile=64, gemm_split_k=4, gemm_portable=True):
        assert (L._ovr.gemm_k_tile, L._ovr.gemm_split_k, L._ovr.gemm_portable) == (64, 4, True)
    assert (L._ovr.gemm_k_tile, L._ovr.gemm_split_k, L._ovr.gemm_portable) == (None, None, False)
