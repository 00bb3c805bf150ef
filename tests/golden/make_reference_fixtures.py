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
    from fxpr_vllm._triton import gemm as ref_gemm

    for name, am, bm, bias, bits in rc.gemm_cases():
        a_d, b_d = am.to(dev), bm.to(dev)
        c = torch.ops.fxpr.gemm_fxp(a_d, b_d, None if bias is None else bias.to(dev), bits, 16)
        out[name] = {"c": c.cpu()}
        # The reference's INTEGER accumulators: its split-K kernel (gemm.py:209-325) sums them
        # into a persistent scratch with integer atomics and the split that arrives last
        # converts and clears them.  With the arrival counters preset far below zero no
        # split is ever "last", so the sums stay in the scratch where they can be read.
        int_dtype = {32: torch.int32, 64: torch.int64}[bits]
        m, n = am.shape[0], bm.shape[1]
        target = ref_gemm._device_sm_count(a_d.device) * ref_gemm._BLOCKS_PER_SM
        c_int_flat, locks_flat = ref_gemm._get_splitk_scratch(a_d.device, int_dtype, target)
        c_int_flat.zero_()
        locks_flat.fill_(-1000)
        ref_gemm._SPLITK_FORCE = 2
        try:
            ref_gemm.gemm_fxp_run(a_d, b_d, None, bits, 16)
            torch.cuda.synchronize()
        finally:
            ref_gemm._SPLITK_FORCE = None
        out[name]["c_int_rows"] = c_int_flat[: m * n].view(m, n)[: rc.GEMM_INT_ROWS].cpu().clone()
        c_int_flat.zero_()
        locks_flat.zero_()
    for name, q, kv, qsl, sl, bt, mq, bits, splits in rc.attention_cases():
        o = torch.empty_like(q, device=dev)
        # The split path allocates its integer totals with torch.zeros on every call
        # (attention.py:838-851) and leaves them filled: record those tensors.
        made = []
        real_zeros = torch.zeros

        def recording_zeros(*args, **kwargs):
            t = real_zeros(*args, **kwargs)
            made.append(t)
            return t

        torch.zeros = recording_zeros
        try:
            torch.ops.fxpr.unified_attention_fxp(q.to(dev), kv.to(dev), o, qsl.to(dev), sl.to(dev), bt.to(dev),
                                                 mq, None, True, None, bits, 16, 0.0, 0, splits)
            torch.cuda.synchronize()
        finally:
            torch.zeros = real_zeros
        out[name] = {"o": o.cpu()}
        ints = [t for t in made if t.dtype in (torch.int32, torch.int64) and t.dim() >= 2 and t.shape[0] == q.shape[0]]
        if splits > 1:
            denom = [t for t in ints if t.dim() == 2]      # creation order: total_denom, then locks
            wv = [t for t in ints if t.dim() == 3]
            assert wv and denom, "integer totals of the split path not found"
            heads = list(rc.ATTN_INT_HEADS)
            heads = [h for h in heads if h < q.shape[1]]
            out[name]["int_heads"] = torch.tensor(heads)
            out[name]["total_wv"] = wv[0][:, heads].cpu().clone()
            out[name]["total_denom"] = denom[0][:, heads].cpu().clone()
    for name, x, r, w in rc.rms_cases():
        rd = r.to(dev).clone()
        y = torch.ops.fxpr.rms_norm_fxp_residual(x.to(dev), rd, w.to(dev), 1e-6)
        out[name] = {"y": y.cpu(), "r": rd.cpu()}
    torch.cuda.synchronize()
    torch.save(out, a.out)
    print("wrote", a.out, "with", len(out) - 1, "cases")


if __name__ == "__main__":
    main()
