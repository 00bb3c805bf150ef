"""Run the REFERENCE plugin's own Triton kernels on this machine's GPU and store their
outputs for the cases in ``reference_cases.py``.

    python tests/golden/make_reference_fixtures.py --ref-path <dir holding fxpr_vllm/> \\
        --out tests/golden/reference_b200.pt

The reference package is not part of this repository: point ``--ref-path`` at a checkout of
Gursukh/vLLM-Triton-Fixed-Point-Reductions.  It must run in a process that has NOT imported
this repository's ``fxpr_vllm`` (both define the ``fxpr`` op library)."""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-path", required=True)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    sys.path.insert(0, a.ref_path)
    sys.path.insert(0, str(Path(__file__).resolve().parent))
    import fxpr_vllm  # the reference
    import reference_cases as rc

    assert "_triton" in [p.name for p in Path(fxpr_vllm.__file__).parent.iterdir()], "not the reference package"
    dev = "cuda"
    out = {"meta": {"gpu": torch.cuda.get_device_name(0), "torch": str(torch.__version__)}}
    for name, x, bits, frac in rc.cast_cases():
        q = torch.ops.fxpr.float_to_fixed(x.to(dev), bits, frac)
        fb = {torch.float16: 16, torch.float32: 32, torch.float64: 64}[x.dtype]
        out[name] = {"q": q.cpu(), "back": torch.ops.fxpr.fixed_to_float(q, fb, frac).cpu()}
    for name, am, bm, bias, bits in rc.gemm_cases():
        c = torch.ops.fxpr.gemm_fxp(am.to(dev), bm.to(dev), None if bias is None else bias.to(dev), bits, 16)
        out[name] = {"c": c.cpu()}
    for name, q, kv, qsl, sl, bt, mq, bits, splits in rc.attention_cases():
        o = torch.empty_like(q, device=dev)
        torch.ops.fxpr.unified_attention_fxp(q.to(dev), kv.to(dev), o, qsl.to(dev), sl.to(dev), bt.to(dev),
                                             mq, None, True, None, bits, 16, 0.0, 0, splits)
        out[name] = {"o": o.cpu()}
    for name, x, r, w in rc.rms_cases():
        rd = r.to(dev).clone()
        y = torch.ops.fxpr.rms_norm_fxp_residual(x.to(dev), rd, w.to(dev), 1e-6)
        out[name] = {"y": y.cpu(), "r": rd.cpu()}
    torch.cuda.synchronize()
    torch.save(out, a.out)
    print("wrote", a.out, "with", len(out) - 1, "cases")


if __name__ == "__main__":
    main()
