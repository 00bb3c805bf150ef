"""Time the REFERENCE plugin's own Triton kernels on this machine's GPU on the benchmark
configurations (same seeded synthetic inputs as ``bench.py``) and print one JSON object.

    python tests/golden/time_reference_kernels.py --ref-path <dir holding fxpr_vllm/> \\
        --synthetic <path to this repository's fxpr_vllm/synthetic.py> [--out file.json]

Runs in a process that has not imported this repository's ``fxpr_vllm`` (both packages define
the ``fxpr`` op library); the input generators are loaded from ``synthetic.py`` by file path.
CUDA events, 5 warm-up calls (the reference autotunes on the first), 20 timed calls."""
from __future__ import annotations

import argparse
import importlib.util
import json
import sys

import torch


def timeit(fn, warm=5, n=20):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3  # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-path", required=True)
    ap.add_argument("--synthetic", required=True)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    sys.path.insert(0, a.ref_path)
    import fxpr_vllm  # noqa: F401  (the reference)
    from fxpr_vllm._triton import gemm as ref_gemm

    spec = importlib.util.spec_from_file_location("fxpr_synthetic", a.synthetic)
    syn = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(syn)
    ops = torch.ops.fxpr
    res = {"gpu": torch.cuda.get_device_name(0)}

    x, r, w = syn.rms_norm_inputs()
    us = timeit(lambda: ops.rms_norm_fxp_residual(x, r, w, 1e-6))
    res["rms_norm_residual_cfg0"] = {"us": us, "GB/s": 4 * x.numel() * 4 / us / 1e3}
    us = timeit(lambda: ops.float_to_fixed(x, 64, 16))
    res["float_to_fixed_i64"] = {"us": us, "GB/s": x.numel() * 12 / us / 1e3}

    am, bm = syn.gemm_inputs()
    flops = 2 * 4096 ** 3
    for kt in (128, 64):
        ref_gemm._BLOCK_K_BY_DTYPE[torch.bfloat16] = kt
        for bits in (64, 32):
            try:
                us = timeit(lambda: ops.gemm_fxp(am, bm, None, bits, 16))
                res[f"gemm_cfg1_ktile{kt}_int{bits}"] = {"us": us, "TFLOP/s": flops / us / 1e6}
            except Exception as e:  # the autotuner may have no configuration for a K-tile
                res[f"gemm_cfg1_ktile{kt}_int{bits}"] = {"error": repr(e)[:200]}
    ref_gemm._BLOCK_K_BY_DTYPE[torch.bfloat16] = 128
    for (M, N, K) in [(64, 4096, 4096), (64, 14336, 4096), (64, 4096, 14336)]:
        a2, b2 = syn.gemm_inputs(M, N, K)
        us = timeit(lambda: ops.gemm_fxp(a2, b2, None, 64, 16))
        res[f"gemm_decode_{M}x{N}x{K}_ktile128_int64"] = {"us": us, "weight GB/s": K * N * 2 / us / 1e3}

    sl = syn.decode_batch_lens()
    q, kv, qsl, seq, bt = syn.paged_attention_inputs(sl, [1] * len(sl))[:5]
    o = torch.empty_like(q)
    nbytes = sum(int(s) for s in sl) * 4096 + 2 * q.numel() * 2
    for s in (0, 1, 4, 8, 16):
        us = timeit(lambda: ops.unified_attention_fxp(q, kv, o, qsl, seq, bt, 1, None, True, None, 64, 16, 0.0, 0, s))
        res[f"decode_attention_cfg2_splits{s}"] = {"us": us, "GB/s": nbytes / us / 1e3}

    pl = syn.prefill_batch_lens()
    q, kv, qsl, seq, bt = syn.paged_attention_inputs(pl, pl, seed=6)[:5]
    o = torch.empty_like(q)
    fl = 8192 * sum(int(l) * (int(l) + 1) for l in pl)
    us = timeit(lambda: ops.unified_attention_fxp(q, kv, o, qsl, seq, bt, max(pl), None, True, None, 64, 16, 0.0, 0, 0), warm=2, n=5)
    res["prefill_attention_cfg3a"] = {"ms": us / 1e3, "TFLOP/s": fl / us / 1e6}

    line = json.dumps(res, indent=1)
    print(line)
    if a.out:
        open(a.out, "w").write(line)


if __name__ == "__main__":
    main()
