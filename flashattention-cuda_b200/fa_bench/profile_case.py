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
    """(callable that launches the workload's kernel once, algorithmic work of a launch: KV bytes for the
    HBM-bound workloads, FLOPs for the tensor-bound ones)."""
    from fa_bench import harness
    case = harness.build(name, device, batch=batch, ctx=ctx)
    work = case["work"]
    return case["step"], (work.kv_bytes if work.bound == "hbm" else work.flops)


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
