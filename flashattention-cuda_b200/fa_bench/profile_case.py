"""Run a few launches of one workload's kernel so that a profiler can be attached to a small, bounded
process (the role of the reference's single-shape loop, bench/regime.py:268-287).

    python flashattention-cuda_b200/fa_bench/profile_case.py --workload paged_gqa_decode_fp16 --launches 4

Prints the CUDA-event time of every launch.  The L2 is flushed before each launch.
"""

from __future__ import annotations

import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import torch  # noqa: E402


def make_step(name, device, batch=None, ctx=None):
    from fa_bench import workloads
    from fa_kernels import gqa_attention
    if name == "paged_gqa_decode_fp16":
        w = workloads.paged_gqa_decode(device, batch=batch or 64)
        fn = lambda: gqa_attention(w["q"], w["k_pool"], w["v_pool"], w["block_table"], w["page_size"], w["seq_lens"],
                                   out_dtype=torch.float16)
        return fn, w["kv_bytes"]
    if name == "causal_prefill_fp16":
        from fa_kernels import attention
        w = workloads.causal_prefill(device, batch=batch or 4)
        fn = lambda: attention(w["q"], w["k"], w["v"], causal=True, out_dtype=torch.float16)
        return fn, w["flops"]
    if name in ("mla_decode_bf16", "mla_decode_fp8"):
        from fa_kernels import mla_attention
        w = workloads.mla_decode(device, batch=batch or 128, latent="bf16" if name.endswith("bf16") else "e4m3")
        fn = lambda: mla_attention(w["q"], w["l_pool"], None, w["block_table"], w["page_size"], w["seq_lens"],
                                   w["kv_lora_rank"], w["scale_l"], out_dtype=torch.bfloat16 if name.endswith("bf16") else torch.float16)
        return fn, w["flops"]
    if name in ("long_decode_fp8", "long_decode_nvfp4"):
        from fa_kernels import fp8_attention, nvfp4_attention
        w = workloads.quantised_long_context_decode(device, fmt="e4m3" if name.endswith("fp8") else "nvfp4",
                                                    batch=batch or 4, ctx=ctx or 1048576)
        if name.endswith("fp8"):
            fn = lambda: fp8_attention(w["q"], w["k_pool"], w["v_pool"], w["block_table"], w["page_size"], w["n_k"],
                                       w["k_scale"], w["v_scale"], out_dtype=torch.float16)
        else:
            fn = lambda: nvfp4_attention(w["q"], w["k_pool"], w["k_micro"], w["v_pool"], w["v_micro"], w["block_table"],
                                         w["page_size"], w["n_k"], w["k_scale"], w["v_scale"], out_dtype=torch.float16)
        return fn, w["kv_bytes"]
    raise SystemExit(f"unknown workload {name!r}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="paged_gqa_decode_fp16")
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--ctx", type=int, default=None, help="context length of the long-context workloads")
    args = ap.parse_args()
    from fa_bench import timing
    dev = torch.device("cuda:0")
    fn, nbytes = make_step(args.workload, dev, args.batch, args.ctx)
    for i, ms in enumerate(timing.time_cuda(fn, warmup=1, iters=args.launches - 1, device=dev)):
        unit = "GFLOP/s" if "prefill" in args.workload or "mla" in args.workload else "GB/s"
        print(f"launch {i + 1}: {ms * 1e3:.1f} us  {nbytes / ms / 1e6:.0f} {unit}")


if __name__ == "__main__":
    main()
