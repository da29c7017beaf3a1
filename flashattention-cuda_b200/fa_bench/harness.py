"""Per-workload measurement rows for every kernel family (the role of the reference's
`python -m bench.harness`, bench/harness.py:101-354: CUDA-event timing with a roofline column).

    python flashattention-cuda_b200/fa_bench/harness.py [--workloads a,b,...] [--iters N]

One JSON line per workload: p10 / p50 / p90 / max milliseconds over CUDA-event samples (L2 flushed before
every launch), the algorithmic work of one launch (fa_bench/roofline.py) and the achieved GB/s or TFLOP/s
as a fraction of the measured peak (MEASURED_PEAKS.json at the repository root when present).  bench.py at
the repository root puts the same rows into its `workloads` array and adds the CPU baseline.
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
if PKG not in sys.path:
    sys.path.insert(0, PKG)

import torch  # noqa: E402

ALL = ["paged_gqa_decode_fp16", "causal_prefill_fp16", "mla_decode_bf16", "mla_decode_fp8", "long_decode_fp8",
       "long_decode_nvfp4"]


def build(name, device, *, batch=None, ctx=None, seq_lens=None, data_seed=None):
    """Seeded inputs of one benchmark configuration and the call that runs its kernel once.
    Returns {"step": callable, "work": roofline.Work, "config": dict, "w": the tensors}."""
    from fa_bench import roofline, workloads
    if name == "paged_gqa_decode_fp16":
        from fa_kernels import gqa_attention
        w = workloads.paged_gqa_decode(device, batch=batch or 64, seq_lens=seq_lens, data_seed=data_seed)
        step = lambda: gqa_attention(w["q"], w["k_pool"], w["v_pool"], w["block_table"], w["page_size"], w["seq_lens"],
                                     out_dtype=torch.float16)
        B = len(w["seq_lens"])
        work = roofline.paged_decode(w["tokens"], H_q=32, H_kv=8, d=128, B=B,
                                     table_entries=sum((n + 15) // 16 for n in w["seq_lens"]))
        cfg = {"workload": name, "batch": B, "h_q": 32, "h_kv": 8, "d": 128, "page_size": 16,
               "ctx": "uniform[1024,8192] seed 2", "kv_tokens": w["tokens"]}
        dtype = "f16"
    elif name == "causal_prefill_fp16":
        from fa_kernels import attention
        w = workloads.causal_prefill(device, batch=batch or 4)
        step = lambda: attention(w["q"], w["k"], w["v"], causal=True, out_dtype=torch.float16)
        B, H, N, d = w["q"].shape
        work = roofline.dense_attention(B, H, N, N, d, causal=True)
        cfg = {"workload": name, "batch": B, "heads": H, "n": N, "d": d, "seed": 1,
               "flops_undiscounted": roofline.dense_attention_full_flops(B, H, N, N, d)}
        dtype = "f16"
    elif name in ("mla_decode_bf16", "mla_decode_fp8"):
        from fa_kernels import mla_attention
        bf = name.endswith("bf16")
        w = workloads.mla_decode(device, batch=batch or 128, latent="bf16" if bf else "e4m3", seq_lens=seq_lens)
        step = lambda: mla_attention(w["q"], w["l_pool"], None, w["block_table"], w["page_size"], w["seq_lens"],
                                     w["kv_lora_rank"], w["scale_l"], out_dtype=torch.bfloat16 if bf else torch.float16)
        B = len(w["seq_lens"])
        work = roofline.mla_decode(w["tokens"], h_q=128, latent_format="bf16" if bf else "e4m3", per_token_scales=not bf, B=B)
        cfg = {"workload": name, "batch": B, "h_q": 128, "dqk": 576, "dv": 512, "page_size": 64,
               "ctx": "uniform[4096,32768] seed 5", "kv_tokens": w["tokens"]}
        dtype = "bf16" if bf else "f16 over e4m3 latent"
    elif name in ("long_decode_fp8", "long_decode_nvfp4"):
        from fa_kernels import fp8_attention, nvfp4_attention
        fp8 = name.endswith("fp8")
        w = workloads.quantised_long_context_decode(device, fmt="e4m3" if fp8 else "nvfp4", batch=batch or 4, ctx=ctx or 1048576)
        if fp8:
            step = lambda: fp8_attention(w["q"], w["k_pool"], w["v_pool"], w["block_table"], w["page_size"], w["n_k"],
                                         w["k_scale"], w["v_scale"], out_dtype=torch.float16)
        else:
            step = lambda: nvfp4_attention(w["q"], w["k_pool"], w["k_micro"], w["v_pool"], w["v_micro"], w["block_table"],
                                           w["page_size"], w["n_k"], w["k_scale"], w["v_scale"], out_dtype=torch.float16)
        B = w["q"].shape[0]
        work = roofline.paged_decode(w["tokens"], H_q=32, H_kv=8, d=128, kv_format="e4m3" if fp8 else "nvfp4",
                                     per_token_scales=fp8, B=B, table_entries=B * (w["n_k"] // 64))
        cfg = {"workload": name, "batch": B, "h_q": 32, "h_kv": 8, "d": 128, "page_size": 64, "ctx": w["n_k"],
               "kv_tokens": w["tokens"], "outlier_channels": "1 % x10"}
        dtype = "f16 over " + ("e4m3" if fp8 else "nvfp4") + " KV"
    else:
        raise SystemExit(f"unknown workload {name!r}")
    return {"step": step, "work": work, "config": cfg, "w": w, "dtype": dtype}


def captured_traffic(name, work):
    """DRAM bytes per launch from the committed ncu captures (profiles/ncu_traffic.json: bytes per unit of
    work measured on a capture of the same kernel, scaled by this launch's units), or None."""
    path = os.path.join(REPO, "profiles", "ncu_traffic.json")
    if not os.path.exists(path):
        return None, None
    with open(path) as f:
        table = json.load(f)
    e = table.get(name)
    if not e:
        return None, None
    units = work.kv_bytes if e["per"] == "kv_byte" else work.flops
    return e["dram_bytes_per_unit"] * units, e["source"]


def measure(name, device, *, iters=20, warmup=3, batch=None, ctx=None, hold_seconds=0.0, case=None):
    """Time one workload's kernel: `iters` CUDA-event samples, L2 flushed and the GPU held busy before
    each.  `hold_seconds` keeps launching afterwards so that a clock sampler sees the GPU under load;
    `case` is a workload already built with `build`."""
    from fa_bench import roofline, timing
    case = case or build(name, device, batch=batch, ctx=ctx)
    t = timing.summary(timing.time_cuda(case["step"], warmup=warmup, iters=iters, device=device))
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < hold_seconds:
        case["step"]()
        torch.cuda.synchronize(device)
    peaks = roofline.measured_peaks()
    roof = roofline.achieved(case["work"], t["p50"] * 1e-3, peaks)
    traffic, src = captured_traffic(name, case["work"])
    roof["traffic"] = traffic
    if src:
        roof["traffic_source"] = src
    row = {"workload": name, "config": case["config"], "dtype": case["dtype"], "p50_ms": t["p50"], "p10_ms": t["p10"],
           "p90_ms": t["p90"], "max_ms": t["max"], "mean_ms": t["mean"], "samples": t["n"], "roofline": roof}
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workloads", default=",".join(ALL))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    for name in args.workloads.split(","):
        print(json.dumps(measure(name, dev, iters=args.iters, batch=args.batch, ctx=args.ctx)), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
