#!/usr/bin/env python
"""Benchmark of the fixed-point reduction hot path on B200.

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line.  A step
is one pass of the headline kernel -- the fixed-point GEMM of the benchmark
configuration (A [4096,4096] ~N(0,1) x B [4096,4096] ~N(0,0.02), bf16, fp32 MMA
partials per K-tile of 64 rounded to Q16.16 and summed in int64, bf16 out) --
over one synthetic batch.  ``value`` is TFLOP/s with inputs resident in HBM,
``e2e`` the same through ``torch.ops.fxpr.gemm_fxp`` with pinned host buffers and
the host<->device copies inside the timed region.  The other configurations
(RMSNorm, decode/prefill attention, log-softmax) are timed briefly and reported
under ``others``.  With N > 1 every rank runs an independent replica (the
kernels have no exchange step): weak scaling, no collective in the data path.

``--impl reference`` times the CPU restatement of the reference's algorithm
(the torch int64 emulation in ``oracle/``; the reference itself has no CPU path
and its Triton kernels cannot run without a GPU) on the host cores, on a bounded
row-sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
PKG = ROOT / "vllm-triton-fixed-point-reductions_b200"
for _p in (str(ROOT), str(PKG)):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "fxp GEMM TFLOP/s + split-K decode attn GB/s (% roofline); bitwise-invariant Y/N"
GEMM = dict(M=4096, N=4096, K=4096, k_tile=64, int_bits=64, frac_bits=16)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL = {"hbm_gbs": 8000.0, "bf16_tflops": 2250.0}
# DRAM bytes of one launch of the headline kernel, from its ncu capture (71.4 MB read + 16.2 MB
# written); a profiler cannot run inside the timed bench, so the captured figure is quoted
GEMM_DRAM_TRAFFIC_BYTES = 87.6e6


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d} | {"source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


def sample_clocks_under_load(fn, index: int, seconds: float = 1.5):
    """Run `fn` back to back for `seconds` while polling SM clock and throttle reasons
    with nvidia-smi (a separate process; polling NVML in-process at a high rate was seen to
    stall kernel launches, so the timed region itself is never sampled)."""
    import subprocess

    q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    gpu_id = str(index)
    if visible:
        ids = visible.split(",")
        if index < len(ids):
            gpu_id = ids[index]
    try:
        proc = subprocess.Popen(["nvidia-smi", f"--id={gpu_id}", f"--query-gpu={q}",
                                 "--format=csv,noheader,nounits", "-lms", "100"],
                                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except Exception as exc:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [f"nvidia-smi unavailable: {exc!r}"]}
    t_end = time.time() + seconds
    i = 0
    while time.time() < t_end:
        for _ in range(20):
            fn(i)
            i += 1
        torch.cuda.synchronize()
    proc.terminate()
    try:
        out, _ = proc.communicate(timeout=3)
    except Exception:
        proc.kill()
        out = ""
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for ln in out.splitlines():
        f = [x.strip() for x in ln.split(",")]
        if len(f) < 6:
            continue
        try:
            sm.append(float(f[0])); mx.append(float(f[1]))
        except ValueError:
            continue
        for n, v in zip(names, f[2:6]):
            if v.lower().startswith("active"):
                reasons.add(n)
    return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "samples": len(sm), "reasons": sorted(reasons),
            "window": f"{seconds} s of back-to-back steps right after the timed region"}


def time_cuda(fn, steps: int, warmup: int, dist=None) -> float:
    """Seconds for `steps` calls of fn (device time via CUDA events on the current
    stream), after `warmup` untimed calls; max over ranks."""
    if dist is not None:
        dist.barrier()          # sets the communicator up now, so the GPU does not idle (and clock
        #                         down) between the warm-up and the timed region
    for i in range(warmup):
        fn(i)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sec = e0.elapsed_time(e1) / 1e3
    if dist is not None:
        t = torch.tensor([sec], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    return sec


# ------------------------------------------------------------------------------
# CPU baseline (oracle) on a bounded sample of the GEMM workload
# ------------------------------------------------------------------------------

def cpu_gemm_baseline(rows: int, repeats: int = 1):
    from oracle import fxp_oracle as orc

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(1)
    a = torch.randn((rows, GEMM["K"]), generator=g).to(torch.bfloat16)
    b = (0.02 * torch.randn((GEMM["K"], GEMM["N"]), generator=g)).to(torch.bfloat16)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.gemm_fxp(a, b, None, GEMM["int_bits"], GEMM["frac_bits"], k_tile=GEMM["k_tile"])
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    flops = 2.0 * rows * GEMM["N"] * GEMM["K"]
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"{rows} of {GEMM['M']} rows of A against the full B, {best:.2f} s "
                      f"(torch CPU int64 emulation of the Q16.16 path)"}


WORKLOAD = ("cfg1 fxp GEMM bf16 4096x4096x4096, K-tile 64, Q16.16 int64, bf16 out (replica per GPU)")


def _reference_gpu_gemm(ref_path: str, steps: int, warm: int):
    """The reference plugin's own Triton GEMM on this GPU, same seeded inputs, K-tile
    forced to 64 like the GPU arm.  Only used when FXPR_REFERENCE_PATH names a checkout of
    the reference (it is not part of this repository); returns seconds for `steps` calls."""
    sys.path[:] = [ref_path] + [q for q in sys.path if q != str(PKG)]
    import fxpr_vllm as ref  # the reference: must have its Triton kernels
    from fxpr_vllm._triton import gemm as ref_gemm

    assert (Path(ref.__file__).parent / "_triton").is_dir(), "FXPR_REFERENCE_PATH is not the reference"
    for dt in list(ref_gemm._BLOCK_K_BY_DTYPE):
        ref_gemm._BLOCK_K_BY_DTYPE[dt] = GEMM["k_tile"]
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    g = torch.Generator(device=dev).manual_seed(1)
    a = torch.randn((GEMM["M"], GEMM["K"]), generator=g, device=dev).to(torch.bfloat16)
    b = (0.02 * torch.randn((GEMM["K"], GEMM["N"]), generator=g, device=dev)).to(torch.bfloat16)
    fn = lambda: torch.ops.fxpr.gemm_fxp(a, b, None, GEMM["int_bits"], GEMM["frac_bits"])
    for _ in range(max(3, warm)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3


def run_reference_arm(args):
    """Rank 0 alone times the reference arm and prints its line; other ranks leave.  The arm is
    the CPU restatement of the reference's algorithm (the reference has no CPU path) on a row
    sample of the same workload, `--steps` timed steps after `--warmup` untimed ones -- or, when
    FXPR_REFERENCE_PATH names a checkout of the reference and a GPU is present, the reference's
    own Triton kernel on the full workload (kind "reference-gpu")."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = max(1, args.steps), max(0, args.warmup)
    flops = 2.0 * GEMM["M"] * GEMM["N"] * GEMM["K"]
    ref_path = os.environ.get("FXPR_REFERENCE_PATH")
    if ref_path and torch.cuda.is_available():
        sec = _reference_gpu_gemm(ref_path, steps, warm)
        value = flops * steps / sec / 1e12
        base = {"value": value, "unit": "TFLOP/s", "cores": 0, "kind": "reference-gpu",
                "sample": "the reference's Triton gemm_fxp on the full 4096^3 workload on this GPU, "
                          "K-tile forced to 64"}
        ms = sec / steps * 1e3
    else:
        rows = 256
        for _ in range(warm):
            cpu_gemm_baseline(rows)
        t0 = time.perf_counter()
        for _ in range(steps):
            one = cpu_gemm_baseline(rows)
        sec = time.perf_counter() - t0
        value = 2.0 * rows * GEMM["N"] * GEMM["K"] * steps / sec / 1e12
        base = dict(one, value=value,
                    sample=f"each step = {rows} of {GEMM['M']} rows of A against the full B "
                           f"(1/16 of the workload; torch CPU int64 emulation of the Q16.16 path)")
        ms = sec / steps * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, **GEMM},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU path of its own (CUDA-only Triton kernels); unless "
                "FXPR_REFERENCE_PATH is set this arm is the torch CPU restatement of its algorithm "
                "from oracle/, so its ratio to the GPU arm compares devices, not kernels "
                "(the reference's Triton kernel on a B200 of this pool: 264 TFLOP/s at K-tile 64)",
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------

def run_gpu_arm(args):
    import fxpr_vllm  # noqa: F401
    from fxpr_vllm import _lib as L
    from fxpr_vllm import synthetic as syn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist_mod.init_process_group("nccl", device_id=dev)
        dist = dist_mod
    peaks = load_peaks()
    steps, warm = max(1, args.steps), max(3, args.warmup)
    M, N, K = GEMM["M"], GEMM["N"], GEMM["K"]
    flops = 2.0 * M * N * K

    # inputs larger than L2: rotate over 4 independent (A, B) sets = 268 MB + outputs
    nsets = 4
    sets = [syn.gemm_inputs(M, N, K, torch.bfloat16, seed=1 + i, device=dev) for i in range(nsets)]
    outs = [None] * nsets

    def gemm_step(i):
        a, b = sets[i % nsets]
        outs[i % nsets] = torch.ops.fxpr.gemm_fxp(a, b, None, GEMM["int_bits"], GEMM["frac_bits"])

    with L.overrides(gemm_k_tile=GEMM["k_tile"], gemm_split_k=1):
        # set-up, not warm-up: one pass over every input set, so that each output slot has had
        # its allocation before anything is timed
        for i in range(nsets):
            gemm_step(i)
        torch.cuda.synchronize()
        # bitwise invariance: split-K sweep and repeats on set 0
        a0, b0 = sets[0]
        ref = torch.ops.fxpr.gemm_fxp(a0, b0, None, 64, 16)
        invariant = True
        for sk in (1, 2, 4, 8, 16):
            with L.overrides(gemm_split_k=sk):
                for _ in range(2):
                    invariant &= bool(torch.equal(ref, torch.ops.fxpr.gemm_fxp(a0, b0, None, 64, 16)))
        sec = time_cuda(gemm_step, steps, warm, dist)
        clocks = sample_clocks_under_load(gemm_step, local)
        L.check_device_status()

        # End to end through the public op with pinned host buffers: every step copies its
        # A and B from the host and its C back.  Copies and the kernel run on four streams (two for the uploads) with
        # two buffer sets, so step i's download and step i + 1's upload overlap step i's GEMM --
        # all of them inside the timed region.
        ha, hb = sets[0][0].cpu().pin_memory(), sets[0][1].cpu().pin_memory()
        hcs = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        das = [torch.empty_like(sets[0][0]) for _ in range(2)]
        dbs = [torch.empty_like(sets[0][1]) for _ in range(2)]
        s_in, s_in_b, s_cmp, s_out = (torch.cuda.Stream(device=dev) for _ in range(4))
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_in_b = [torch.cuda.Event() for _ in range(2)]
        ev_cmp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def e2e_step(i):
            k = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_cmp[k])                 # the GEMM that last read this buffer set
                das[k].copy_(ha, non_blocking=True)
                ev_in[k].record(s_in)
            with torch.cuda.stream(s_in_b):                # A and B go up on two streams
                s_in_b.wait_event(ev_cmp[k])
                dbs[k].copy_(hb, non_blocking=True)
                ev_in_b[k].record(s_in_b)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in[k])
                s_cmp.wait_event(ev_in_b[k])
                c = torch.ops.fxpr.gemm_fxp(das[k], dbs[k], None, GEMM["int_bits"], GEMM["frac_bits"])
                ev_cmp[k].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[k])
                s_out.wait_event(ev_out[k])                # the download that last wrote this host buffer
                c.record_stream(s_out)
                hcs[k].copy_(c, non_blocking=True)
                ev_out[k].record(s_out)

        def e2e_run(n, first):
            cur = torch.cuda.current_stream(dev)
            for st in (s_in, s_in_b, s_cmp, s_out):
                st.wait_stream(cur)
            for i in range(n):
                e2e_step(first + i)
            for st in (s_in, s_in_b, s_cmp, s_out):
                cur.wait_stream(st)

        e2e_steps = max(4, min(steps, 10))
        e2e_run(4, 0)
        # three repeats, median reported (host-side copies vary from run to run on a shared box)
        e2e_secs = sorted(time_cuda(lambda i: e2e_run(e2e_steps, 0) if i == 1 else None, 1, 1, dist)
                          for _ in range(3))
        sec_e2e = e2e_secs[1]
        hc = hcs[(e2e_steps - 1) % 2]
    e2e_ok = bool(torch.equal(hc, ref.cpu()))

    value = world * flops * steps / sec / 1e12
    per_gpu = flops * steps / sec / 1e12
    peak = peaks["bf16_tflops"]
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": sec / steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, **GEMM,
                   "l2": f"rotating {nsets} input sets (268 MB) > 126 MB L2",
                   "seed": "1..4"},
        "bitwise_invariant": "Y" if invariant else "N",
        "invariance_checked": "split-K {1,2,4,8,16} x 2 repeats, identical bf16 outputs",
        "e2e": {"value": world * flops * e2e_steps / sec_e2e / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": ha.numel() * 2 + hb.numel() * 2,
                "d2h_bytes_per_step": hc.numel() * 2, "matches_resident_run": e2e_ok,
                "repeats_TFLOP/s": [world * flops * e2e_steps / t_ / 1e12 for t_ in e2e_secs],
                "how": "uploads (A and B on two streams), GEMM and download of consecutive steps overlapped "
                       "(two buffer sets); every step still moves all of its bytes"},
        "gpu_launches": steps,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                     "frac": per_gpu / peak, "traffic": GEMM_DRAM_TRAFFIC_BYTES,
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of "
                                       "this kernel on this workload: A and B once (67.1 MB) plus the part "
                                       "of C that left L2 during the launch",
                     "peak_source": f"{peaks['source']} cuBLAS bf16 burst",
                     "frac_of_nominal_2250": per_gpu / NOMINAL["bf16_tflops"],
                     "algorithmic": "2*M*N*K = 137.44 GFLOP per launch"},
    }
    if not args.skip_others:
        line["others"] = bench_others(dev, peaks, L, syn)
    if "others" in line and "decode_attention_cfg2" in line["others"]:
        # the second half of the metric's name, lifted out of `others` (per GPU; replicas do not add)
        auto = line["others"]["decode_attention_cfg2"]["auto"]
        line["decode_attention"] = {"metric": "split-K decode attention GB/s (cfg2: batch 64, ctx U[512,8192])",
                                    "value": auto["GB/s"], "unit": "GB/s", "us": auto["us"],
                                    "frac_hbm_measured": auto["frac_hbm_measured"],
                                    "bitwise_invariant": line["others"]["decode_attention_cfg2"]["bitwise_invariant"]}
    if not args.skip_model:
        line.setdefault("others", {})["llama3_8b_decode_cfg4"] = bench_llama(dev, dist, world, peaks)
    if rank == 0:
        if not args.skip_cpu:
            line["cpu_baseline"] = cpu_gemm_baseline(256)
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def _digest(t: torch.Tensor) -> int:
    """Position-sensitive 64-bit checksum of a 16-bit tensor's bit patterns."""
    v = t.contiguous().view(torch.int16).reshape(-1).to(torch.int64)
    w = torch.arange(v.numel(), device=v.device, dtype=torch.int64) % 65521 + 1
    return int((v * w).sum().item())


def bench_llama(dev, dist, world, peaks, batch=64, prompt_len=1024, gen=256):
    """cfg4: random-init Llama-3-8B-shaped decoder, 64 sequences x 1024 prompt tokens, 256
    greedy decode steps, tensor parallel over all ranks of the job (TP = n_gpus) with the
    integer all-reduce.  The logits digests must be the same for every TP degree."""
    from fxpr_vllm.llama_decoder import DecoderConfig, DistGroup, LlamaDecoder, LocalGroup

    cfg = DecoderConfig()
    group = DistGroup() if dist is not None else LocalGroup(1)
    t0 = time.time()
    model = LlamaDecoder(cfg, group, dev, seed=0, max_seqs=batch, max_len=prompt_len + gen)
    g = torch.Generator().manual_seed(7)
    prompts = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=g).to(dev)
    torch.cuda.synchronize()
    build_s = time.time() - t0

    def timed(fn):
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return out, float(ms.item())

    peer_setup_error = None
    if dist is not None and os.environ.get("FXPR_BENCH_NCCL_EXCHANGE") != "1":
        # decode-sized batches exchange through the peer-memory reduce + norm kernel (same bits);
        # the prefill below is too large for its buffers and takes the ncclAllReduce path
        try:
            model.enable_peer_reduce()
        except RuntimeError as e:            # raised on every rank or on none: the run goes on with ncclAllReduce
            model.peer = None
            peer_setup_error = repr(e)[:200]
    logits, prefill_ms = timed(lambda: model.prefill(prompts))
    d_prefill = _digest(logits)
    state = {"tok": model.greedy(logits), "logits": logits}
    peer_note = None
    if model.peer is not None:
        # one eager decode step through each exchange before anything is timed: the peer-memory
        # kernel must reproduce the ncclAllReduce path bit for bit on every rank and report no
        # timed-out wait, else the run continues on ncclAllReduce (the default exchange)
        from fxpr_vllm import _lib as L

        peer, model.peer = model.peer, None
        want = model.decode_step(state["tok"], prompt_len)
        model.peer = peer
        got = model.decode_step(state["tok"], prompt_len)
        ok = bool(torch.equal(want, got))
        try:
            L.check_device_status(dev)
        except RuntimeError:
            ok = False
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) != 1:
            model.peer = None
            peer_note = "peer-memory exchange failed its self-check on this box; ncclAllReduce used"

    def decode_all():
        for step in range(gen):
            state["logits"] = model.decode_step(state["tok"], prompt_len + step)
            state["tok"] = model.greedy(state["logits"])

    graph_error = None
    try:
        model.capture_decode(state["tok"], prompt_len)

        def decode_all_graph():
            for _ in range(gen):
                model.replay_decode()
            state["logits"] = model.last_logits()

        _, decode_ms = timed(decode_all_graph)
        state["tok"] = model._g_tok
        launch = "one CUDA graph per decode step"
    except Exception as e:  # capture not possible (for example an old NCCL): time the eager loop
        graph_error = repr(e)[:200]
        _, decode_ms = timed(decode_all)
        launch = "python-launched ops"
    tp_scaling = None
    if dist is not None and graph_error is None:
        tp_scaling = _tp_scaling(model, cfg, dev, dist, world, timed, state, prompts, prompt_len, gen,
                                 decode_ms / gen)
    weights_gb = (cfg.layers * (cfg.hidden * (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim
                                + cfg.q_heads * cfg.head_dim * cfg.hidden + 3 * cfg.hidden * cfg.ffn)
                  + cfg.hidden * cfg.vocab) * 2 / 1e9
    kv_gb = batch * (prompt_len + gen / 2) * cfg.layers * 2 * cfg.kv_heads * cfg.head_dim * 2 / 1e9
    step_ms = decode_ms / gen
    return {
        "tp": world, "decode_tokens_per_s": batch * gen / (decode_ms / 1e3), "decode_ms_per_step": step_ms,
        "prefill_ms": prefill_ms, "prefill_tokens_per_s": batch * prompt_len / (prefill_ms / 1e3),
        "algorithmic_GB_per_step": weights_gb + kv_gb,
        "frac_hbm_measured": (weights_gb + kv_gb) / world / (step_ms / 1e3) / peaks["hbm_gbs"],
        "logits_digest_prefill": d_prefill, "logits_digest_last": _digest(state["logits"]),
        "last_tokens_digest": int((state["tok"] * (torch.arange(batch, device=dev) + 1)).sum().item()),
        "build_s": build_s,
        "launch": launch, "graph_error": graph_error, "tp_scaling": tp_scaling,
        "exchange": ("single GPU" if dist is None else
                     "peer-memory reduce+norm kernel" if model.peer is not None else "ncclAllReduce + norm kernel"),
        "exchange_note": peer_note or peer_setup_error,
        "note": "digests are equal across TP degrees when the integer all-reduce keeps the logits "
                "bit-identical",
    }


def _tp_scaling(model, cfg, dev, dist, world, timed, state, prompts, prompt_len, gen, step_ms, short=64):
    """How the decode step divides at TP = world.  The last `short` positions are decoded again
    (deterministic: same tokens, same KV prefix) with (a) ncclAllReduce + norm kernel, (b) the
    peer-memory reduce + norm kernel -- their logits digests must agree -- and (c) no exchange at
    all (wrong results, same kernels), which gives the collective share; a TP = 1 copy of the
    model on this GPU gives the speed-up.  Runs after the headline digests are taken."""
    from fxpr_vllm.llama_decoder import LlamaDecoder, LocalGroup

    start = prompt_len + gen - short
    tok0 = state["tok"].clone()

    def run():
        model.capture_decode(tok0, start)

        def replay():
            for _ in range(short):
                model.replay_decode()

        _, ms = timed(replay)
        return ms / short, _digest(model.last_logits())

    peer, model.peer = model.peer, None
    nccl_ms, d_nccl = run()
    model.peer = peer
    peer_ms, d_peer = run() if peer is not None else (None, None)
    model.group.skip_collectives = True
    try:
        no_coll, _ = run()
    finally:
        model.group.skip_collectives = False
    del model._graph
    one = LlamaDecoder(cfg, LocalGroup(1), dev, seed=0, max_seqs=prompts.shape[0], max_len=prompt_len + gen)
    tok = one.greedy(one.prefill(prompts))
    one.capture_decode(tok, prompt_len)

    def replay_one():
        for _ in range(short):
            one.replay_decode()

    _, ms1 = timed(replay_one)
    tp1 = ms1 / short
    del one
    torch.cuda.empty_cache()
    return {"tp": world, "ms_per_step": step_ms,
            "exchange": "peer-memory reduce+norm kernel" if peer is not None else "ncclAllReduce + norm kernel",
            "ms_per_step_nccl_exchange": nccl_ms, "ms_per_step_peer_exchange": peer_ms,
            "digests_equal_nccl_vs_peer": None if peer is None else bool(d_nccl == d_peer),
            "ms_per_step_without_collectives": no_coll,
            "collective_share": max(0.0, 1.0 - no_coll / step_ms),
            "collective_share_nccl_exchange": max(0.0, 1.0 - no_coll / nccl_ms),
            "tp1_ms_per_step": tp1, "speedup_vs_tp1": tp1 / step_ms,
            "how": f"{short} replays each over the last {short} positions; 'without collectives' skips the "
                   "exchanges (results discarded); TP=1 is the same model unsharded on this GPU"}


def bench_others(dev, peaks, L, syn):
    """Short timings of the other configurations (device time, L2 flushed by rotating
    inputs where they are smaller than L2)."""
    res = {}
    hbm = peaks["hbm_gbs"]

    def t(fn, steps=10, warm=3):
        return time_cuda(fn, steps, warm) / steps

    # cfg0: RMSNorm + residual, fp32 [2048, 4096]
    sets = [syn.rms_norm_inputs(seed=10 + i, device=dev) for i in range(4)]
    sec = t(lambda i: torch.ops.fxpr.rms_norm_fxp_residual(*sets[i % 4][:2], sets[i % 4][2], 1e-6))
    byts = 4 * 2048 * 4096 * 4 + 4096 * 4
    res["rms_norm_residual_cfg0"] = {"us": sec * 1e6, "GB/s": byts / sec / 1e9,
                                     "frac_hbm_measured": byts / sec / 1e9 / hbm}

    # cfg3b: log-softmax fp32 [256, 128256]
    lsets = [syn.logits_inputs(seed=20 + i, device=dev) for i in range(2)]
    sec = t(lambda i: torch.ops.fxpr.log_softmax_fxp(lsets[i % 2], 16))
    byts = 2 * 256 * 128256 * 4
    res["log_softmax_cfg3b"] = {"us": sec * 1e6, "GB/s": byts / sec / 1e9,
                                "frac_hbm_measured": byts / sec / 1e9 / hbm}

    # casts: fp32 -> int64 -> fp32 on [2048, 4096]
    x = sets[0][0]
    sec = t(lambda i: torch.ops.fxpr.float_to_fixed(sets[i % 4][0], 64, 16))
    byts = x.numel() * 12
    res["float_to_fixed_i64"] = {"us": sec * 1e6, "GB/s": byts / sec / 1e9,
                                 "frac_hbm_measured": byts / sec / 1e9 / hbm}

    # cfg1 at the reference's own K-tile (128): 128 x 256 output tiles
    ga, gb = syn.gemm_inputs(device=dev)
    with L.overrides(gemm_k_tile=128, gemm_split_k=1):
        sec = t(lambda i: torch.ops.fxpr.gemm_fxp(ga, gb, None, 64, 16), steps=20, warm=5)
    res["gemm_cfg1_ktile128"] = {"us": sec * 1e6, "TFLOP/s": 2.0 * 4096 ** 3 / sec / 1e12,
                                 "frac_tensor_measured": 2.0 * 4096 ** 3 / sec / 1e12 / peaks["bf16_tflops"]}

    # cfg4's decode GEMM shapes (M = 64, K-tile 128), kernel-only: 20 launches in a CUDA graph
    def graph_us(fn, n=20, reps=5):
        fn()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(n):
                fn()
        g.replay()
        return time_cuda(lambda i: g.replay(), reps, 1) / (n * reps) * 1e6

    shapes = {"qkv 64x6144x4096": (64, 6144, 4096), "o_proj 64x4096x4096": (64, 4096, 4096),
              "gate_up 64x28672x4096": (64, 28672, 4096), "down 64x4096x14336": (64, 4096, 14336),
              "lm_head 64x128256x4096": (64, 128256, 4096)}
    dec = {}
    for name, (m_, n_, k_) in shapes.items():
        xa, wb = syn.gemm_inputs(m_, n_, k_, device=dev, seed=40)
        with L.overrides(gemm_k_tile=128):
            us = graph_us(lambda: torch.ops.fxpr.gemm_fxp(xa, wb, None, 64, 16))
        dec[name] = {"us": us, "weights_GB/s": k_ * n_ * 2 / us / 1e3,
                     "frac_hbm_measured": k_ * n_ * 2 / us / 1e3 / hbm}
        del xa, wb
    res["gemm_decode_shapes_cfg4"] = dec

    # cfg2: paged decode attention, batch 64, ctx U[512, 8192]
    lens = syn.decode_batch_lens()
    q, kv, qsl, sl, bt = syn.paged_attention_inputs(lens, [1] * len(lens), device=dev)
    o = torch.empty_like(q)
    byts = sum(lens) * 4096 + 2 * q.numel() * 2
    dec = {}
    ref = None
    inv = True
    for splits in (0, 1, 4, 8, 16):
        def step(i, s=splits):
            torch.ops.fxpr.unified_attention_fxp(q, kv, o, qsl, sl, bt, 1, None, True, None, 64, 16,
                                                 0.0, 0, s)
        # ten launches in one CUDA graph, replayed three times: device time without the gaps a
        # short Python loop leaves in front of a 250 us kernel (the 1.08 GB of KV exceeds L2)
        sec = graph_us(lambda s=splits: step(0, s), n=10, reps=3) / 1e6
        dec["auto" if splits == 0 else f"splits{splits}"] = {"us": sec * 1e6, "GB/s": byts / sec / 1e9,
                                  "frac_hbm_measured": byts / sec / 1e9 / hbm}
        cur = o.clone()
        if ref is None:
            ref = cur
        inv &= bool(torch.equal(ref, cur))
    dec["bitwise_invariant"] = "Y" if inv else "N"
    dec["algorithmic_bytes"] = byts
    res["decode_attention_cfg2"] = dec

    # cfg3a: varlen causal prefill, 16 seqs U[128, 4096]
    plens = syn.prefill_batch_lens()
    q, kv, qsl, sl, bt = syn.paged_attention_inputs(plens, plens, device=dev, seed=6)
    o = torch.empty_like(q)
    fl = 8192.0 * sum(l * (l + 1) for l in plens)

    def pstep(i):
        torch.ops.fxpr.unified_attention_fxp(q, kv, o, qsl, sl, bt, max(plens), None, True, None, 64,
                                             16, 0.0, 0, 1)
    sec = t(pstep, steps=3, warm=1)
    o_tc = o.clone()
    from fxpr_vllm import _native as nat
    with L.overrides(attn_flags=nat.ATTN_NO_TCGEN05):
        sec_mma = t(pstep, steps=3, warm=1)
    res["prefill_attention_cfg3a"] = {"ms": sec * 1e3, "TFLOP/s": fl / sec / 1e12,
                                      "frac_tensor_measured": fl / sec / 1e12 / peaks["bf16_tflops"],
                                      "route": "tcgen05 + TMEM + TMA (attn_tc_prefill_kernel)",
                                      "mma_sync_kernel_ms": sec_mma * 1e3,
                                      "routes_bit_identical": bool(torch.equal(o_tc, o))}
    L.check_device_status()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-others", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-model", action="store_true", help="skip the cfg4 decoder run")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
