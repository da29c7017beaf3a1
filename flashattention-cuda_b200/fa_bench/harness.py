"""Per-workload measurement rows for every kernel family (the role of the reference's
`python -m bench.harness`, bench/harness.py:101-354: CUDA-event timing against a CPU/torch baseline
with a roofline column).

    python flashattention-cuda_b200/fa_bench/harness.py [--workloads a,b,...] [--iters N] [--cpu-seconds S]

One JSON line per workload: p50 / min microseconds, achieved GB/s or TFLOP/s, fraction of the measured
peak (MEASURED_PEAKS.json at the repository root when present), and the reference's CPU path (torch
SDPA through oracle/cpu_reference.py) timed on a bounded sample of the same inputs.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
REPO = os.path.dirname(PKG)
for p_ in (PKG, REPO):
    if p_ not in sys.path:
        sys.path.insert(0, p_)

import torch  # noqa: E402

ALL = ["paged_gqa_decode_fp16", "long_decode_fp8", "long_decode_nvfp4", "causal_prefill_fp16", "mla_decode_bf16",
       "mla_decode_fp8"]


def peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def cpu_sample(name, w, seconds):
    """Time the reference CPU path on a bounded sample; returns (work_done, seconds, description)."""
    from oracle import cpu_reference as R
    t_used, work = 0.0, 0.0
    if name == "paged_gqa_decode_fp16":
        kp, vp, bt, q = w["k_pool"].cpu(), w["v_pool"].cpu(), w["block_table_host"], w["q"].float().cpu()
        n_done = 0
        for b, n in enumerate(w["seq_lens"]):
            k = R.gather_dense(kp, bt[b], w["page_size"], n).float()
            v = R.gather_dense(vp, bt[b], w["page_size"], n).float()
            t0 = time.perf_counter()
            R.sdpa_reference_gqa(q[b:b + 1], k, v)
            t_used += time.perf_counter() - t0
            work += n * 2 * kp.shape[2] * kp.shape[3] * 2
            n_done += 1
            if t_used > seconds:
                break
        return work, t_used, f"{n_done} sequences, fp32 SDPA on dense KV"
    if name.startswith("long_decode"):
        from fa_kernels import paged as P
        n = 131072                                           # one (sequence, kv head) slice of 128K keys, scaled linearly
        bt = w["block_table"][:1, : n // w["page_size"]].contiguous()
        if name.endswith("fp8"):
            k = P.dequantize_fp8_e4m3(P.paged_gather(w["k_pool"], bt, w["page_size"], n), P.paged_gather(w["k_scale"].unsqueeze(-1), bt, w["page_size"], n)[..., 0])
            v = P.dequantize_fp8_e4m3(P.paged_gather(w["v_pool"], bt, w["page_size"], n), P.paged_gather(w["v_scale"].unsqueeze(-1), bt, w["page_size"], n)[..., 0])
            per_tok = 2 * 8 * (128 + 4)
        else:
            k = P.dequantize_nvfp4(P.paged_gather(w["k_pool"], bt, w["page_size"], n), P.paged_gather(w["k_micro"], bt, w["page_size"], n), w["k_scale"])
            v = P.dequantize_nvfp4(P.paged_gather(w["v_pool"], bt, w["page_size"], n), P.paged_gather(w["v_micro"], bt, w["page_size"], n), w["v_scale"])
            per_tok = 2 * 8 * 72
        k, v, q = k.cpu(), v.cpu(), w["q"][:1].float().cpu()
        reps = 0
        while t_used < seconds:
            t0 = time.perf_counter()
            R.sdpa_reference_gqa(q, k, v)
            t_used += time.perf_counter() - t0
            reps += 1
        return reps * n * per_tok, t_used, f"{reps} passes over the first 131072 keys of sequence 0 (dequantised outside the timing)"
    if name == "causal_prefill_fp16":
        q, k, v = (w[x][:1, :2].float().cpu() for x in ("q", "k", "v"))
        reps = 0
        while t_used < seconds:
            t0 = time.perf_counter()
            R.sdpa_reference(q, k, v, causal=True)
            t_used += time.perf_counter() - t0
            reps += 1
        n, d = q.shape[2], q.shape[3]
        return reps * 2 * 2 * d * n * (n + 1), t_used, f"{reps} passes over 2 of {w['q'].shape[0] * w['q'].shape[1]} heads, fp32 SDPA"
    if name.startswith("mla_decode"):
        from fa_kernels import paged as P
        n = min(w["seq_lens"][0], 8192)
        bt = w["block_table"][:1].contiguous()
        lat = P.paged_gather(w["l_pool"], bt, w["page_size"], n)
        if name.endswith("fp8"):
            lat = P.dequantize_fp8_e4m3(lat, P.paged_gather(w["scale_l"].unsqueeze(-1), bt, w["page_size"], n)[..., 0])
        lat, q = lat.float().cpu(), w["q"][:1].float().cpu()
        reps = 0
        while t_used < seconds:
            t0 = time.perf_counter()
            R.sdpa_reference_mla_dequantised(q, lat, w["kv_lora_rank"])
            t_used += time.perf_counter() - t0
            reps += 1
        return reps * 2 * q.shape[1] * (q.shape[3] + w["kv_lora_rank"]) * n, t_used, f"{reps} passes over the first {n} keys of sequence 0"
    raise ValueError(name)


def run(name, iters, cpu_seconds, ctx=None, batch=None):
    from fa_bench import timing, workloads
    from fa_bench.profile_case import make_step
    dev = torch.device("cuda:0")
    hbm, tflops, src = peaks()
    holder = {}
    orig = {}
    # capture the workload dict that make_step builds (for the CPU sample) by wrapping the builders
    for fn_name in ("paged_gqa_decode", "quantised_long_context_decode", "causal_prefill", "mla_decode"):
        orig[fn_name] = getattr(workloads, fn_name)

        def wrap(f):
            def inner(*a, **k):
                holder["w"] = f(*a, **k)
                return holder["w"]
            return inner
        setattr(workloads, fn_name, wrap(orig[fn_name]))
    try:
        fn, work = make_step(name, dev, batch, ctx)
    finally:
        for k_, v_ in orig.items():
            setattr(workloads, k_, v_)
    t = timing.summary(timing.time_cuda(fn, warmup=3, iters=iters, device=dev))
    tensor_bound = "prefill" in name or "mla" in name
    achieved = work / (t["p50"] * 1e-3) / (1e12 if tensor_bound else 1e9)
    peak = tflops if tensor_bound else hbm
    row = {"workload": name, "p50_us": t["p50"] * 1e3, "min_us": t["min"] * 1e3, "algorithmic_work": work,
           "roofline": {"bound": "tensor" if tensor_bound else "hbm", "achieved": achieved, "peak": peak,
                        "unit": "TFLOP/s" if tensor_bound else "GB/s", "frac": achieved / peak, "peak_source": src}}
    if cpu_seconds > 0:
        done, secs, desc = cpu_sample(name, holder["w"], cpu_seconds)
        row["cpu_baseline"] = {"value": done / secs / (1e12 if tensor_bound else 1e9), "unit": row["roofline"]["unit"],
                               "cores": torch.get_num_threads(), "kind": "port", "sample": desc}
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workloads", default=",".join(ALL))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--cpu-seconds", type=float, default=3.0)
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    args = ap.parse_args()
    for name in args.workloads.split(","):
        print(json.dumps(run(name, args.iters, args.cpu_seconds, args.ctx, args.batch)), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
