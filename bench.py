"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one pass of the hot path over one batch of seeded synthetic input.  The default workload
is the paged GQA decode configuration (fp16 KV, batch 64 per GPU, 32 query / 8 KV heads, d=128,
context lengths uniform in [1024, 8192], 16-token pages, shuffled block table); the metric is the
KV bytes streamed per second.  Rank 0 prints one JSON line.  Under torchrun every rank owns its own
batch (weak scaling, no data-path collective), times on its own device with CUDA events, and the
slowest rank defines the step time.

`--impl reference` times the reference project's CPU implementation of the same path (torch SDPA
through the wrappers of its fa_kernels/reference.py, restated in oracle/cpu_reference.py) on the
host cores of this machine.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(REPO, "flashattention-cuda_b200"))
sys.path.insert(0, REPO)

import torch  # noqa: E402

METRIC = {"metric": "decode_kv_gbs", "unit": "GB/s", "higher_is_better": True}


def measured_peaks():
    """HBM GB/s and bf16 TFLOP/s measured on this pool (MEASURED_PEAKS.json), else the documented
    fallback of an earlier measurement."""
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            self.result = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                           "samples": len(sm)}


# --------------------------------------------------------------------------------------------------
def build_workload(name, device, rank):
    from fa_bench import workloads
    if name == "paged_gqa_decode_fp16":
        # weak scaling: every GPU gets the same amount of work (the seed-2 context lengths and page
        # permutation of the single-GPU configuration) over its own K, V and q values
        w = workloads.paged_gqa_decode(device, seed=2, data_seed=2 + 1000 * rank)
        w["describe"] = {"workload": "paged_gqa_decode_fp16", "batch_per_gpu": 64, "h_q": 32, "h_kv": 8, "d": 128,
                         "page_size": 16, "ctx": "uniform[1024,8192] seed 2", "kv_tokens_per_gpu": w["tokens"]}
        return w
    raise SystemExit(f"unknown workload {name!r}")


def run_ours(args):
    import torch.distributed as dist
    from fa_bench import timing
    from fa_kernels import _decode, _lib, gqa_attention

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    _lib.load()                                     # no library, no benchmark

    w = build_workload(args.workload, device, rank)
    page = w["page_size"]
    lens = w["seq_lens"]

    def step():
        return gqa_attention(w["q"], w["k_pool"], w["v_pool"], w["block_table"], page, lens,
                             out_dtype=torch.float16)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---- device-resident throughput: K steps, each one kernel launch bracketed by events --------
    for _ in range(max(args.warmup, 3)):
        timing.flush_l2(device)
        step()
    barrier()
    with ClockSampler(local_rank) as clocks:
        t_wall0 = time.perf_counter()
        step_ms = []
        for _ in range(args.steps):
            timing.flush_l2(device)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            e1.synchronize()
            step_ms.append(e0.elapsed_time(e1))
        barrier()
        # keep the GPU busy long enough for the 200 ms clock sampler to see it under load
        while time.perf_counter() - t_wall0 < 1.0:
            step()
        torch.cuda.synchronize(device)
    ms_per_step = sum(step_ms) / len(step_ms)

    # ---- roofline: every timed step is exactly one launch of the decode kernel, so the kernel's
    # average launch duration over the timed region is the step time of this rank
    kernel_ms = ms_per_step

    # ---- end to end through the public API with host buffers ------------------------------------
    # One C-ABI call per step (fa_paged_decode_host through fa_kernels.HostDecodeStep): q, block table and the
    # sequence lengths come from pinned host memory, the plan is rebuilt for the step's lengths (a serving
    # step has new lengths), the output lands in pinned host memory; the KV cache is resident device state.
    from fa_kernels import HostDecodeStep
    q_host = w["q"].cpu().pin_memory()
    bt_host = w["block_table_host"].pin_memory()
    lens_host = torch.tensor(lens, dtype=torch.int32).pin_memory()
    out_host = torch.empty(w["q"].shape, dtype=torch.float16).pin_memory()
    B_, Hq_, Nq_, d_ = w["q"].shape
    host_step = HostDecodeStep(w["k_pool"], w["v_pool"], page, B_, Hq_, Nq_, d_, bt_host.shape[1], out_dtype=torch.float16)
    e2e_ms = []
    for i in range(3 + args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        timing.flush_l2(device)
        torch.cuda.synchronize(device)
        e0.record()
        host_step(q_host, bt_host, lens_host, out_host)
        e1.record()
        e1.synchronize()
        if i >= 3:
            e2e_ms.append(e0.elapsed_time(e1))
    # the same inputs through the device-tensor API give the same bytes
    check = gqa_attention(w["q"], w["k_pool"], w["v_pool"], w["block_table"], page, lens, out_dtype=torch.float16)
    assert torch.equal(check.cpu(), out_host), "host-buffer step and device-tensor API disagree"
    items_bytes = _decode.plan(tuple(lens), max(lens), B_, w["k_pool"].shape[2], (Hq_ // w["k_pool"].shape[2]) * Nq_, page, device)[0].numel() * 4
    e2e_ms_mean = sum(e2e_ms) / len(e2e_ms)
    h2d = q_host.numel() * 2 + bt_host.numel() * 4 + items_bytes     # lengths are read by the host planner
    d2h = out_host.numel() * 2

    # ---- reduce over ranks (slowest rank defines the step) --------------------------------------
    stats = torch.tensor([ms_per_step, e2e_ms_mean, float(w["kv_bytes"]), kernel_ms], device=device, dtype=torch.float64)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms_per_step, e2e_ms_mean, kernel_ms = mx[0].item(), mx[1].item(), mx[3].item()
        total_kv_bytes = sm[2].item()
    else:
        total_kv_bytes = float(w["kv_bytes"])

    if rank == 0:
        peaks = measured_peaks()
        achieved = w["kv_bytes"] / (kernel_ms * 1e-3) / 1e9
        line = dict(METRIC)
        line.update({
            "value": total_kv_bytes / (ms_per_step * 1e-3) / 1e9,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": dict(w["describe"], l2="flushed between steps outside the event windows: 512 MB overwritten, then 256 MB read so that the cold L2 holds no dirty lines",
                           sharding="one independent batch per GPU, no collective"),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "algorithmic_bytes": w["kv_bytes"], "kernel_ms": kernel_ms,
                         "frac_of_nominal_8TBs": achieved / 8000.0, "traffic": TRAFFIC_BYTES_PER_LAUNCH},
            "e2e": {"value": total_kv_bytes / (e2e_ms_mean * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms_mean,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "one fa_paged_decode_host call per step (fa_kernels.HostDecodeStep): q, block table and the "
                            "step's split plan copied from pinned host memory, output copied back to pinned host memory; "
                            "the KV cache is resident device state"},
            "gpu_launches": args.steps,
            "clocks": clocks.result,
            "cpu_baseline": cpu_baseline(w, bounded_s=20.0),
        })
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_long_decode(args):
    """Quantised-KV long-context decode (B=4, context 1 048 576, page 64), sharded by KV range: rank r owns the
    keys of logical pages [r*P/N, (r+1)*P/N) of every sequence in its own pool; one step = local decode +
    one NCCL all-gather of (O, LSE) + merge on every rank.  Strong scaling: the context is fixed."""
    import torch.distributed as dist
    from fa_bench import timing, workloads
    from fa_kernels import _lib, fp8_attention, nvfp4_attention
    from fa_kernels.distributed import kv_range_decode, kv_range_shards

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    _lib.load()
    fmt = "e4m3" if args.workload.endswith("fp8") else "nvfp4"
    ctx, page = args.ctx, 64
    kb, ke = kv_range_shards(ctx, page, world)[rank]
    # every rank draws its own shard of the same distribution (seed 3 + rank); q is common (seed 3)
    w = workloads.quantised_long_context_decode(device, fmt=fmt, ctx=ke - kb, seed=3 + rank)
    gq = torch.Generator(device=device).manual_seed(3)
    q = torch.randn(4, 32, 1, 128, device=device, generator=gq).half()
    if fmt == "e4m3":
        fn, before, after = fp8_attention, (w["k_pool"], w["v_pool"], w["block_table"], page), (w["k_scale"], w["v_scale"])
    else:
        fn = nvfp4_attention
        before = (w["k_pool"], w["k_micro"], w["v_pool"], w["v_micro"], w["block_table"], page)
        after = (w["k_scale"], w["v_scale"])

    def step(qq=q):
        if world == 1:
            return fn(qq, *before, ke - kb, *after, out_dtype=torch.float16)
        return kv_range_decode(fn, qq, before, after, local_n_k=ke - kb, key_begin=kb, out_dtype=torch.float16)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(args.warmup, 3)):
        timing.flush_l2(device)
        step()
    barrier()
    # One step is three launches (decode, all-gather, merge) of a few hundred microseconds in total, so the
    # host gaps between them matter: replay the step from a CUDA graph (NCCL collectives can be captured).
    run_step, graphed = step, False
    if world > 1 and not args.no_graph:
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                for _ in range(2):
                    step()
            torch.cuda.current_stream(device).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_out = step()
            run_step, graphed = graph.replay, True
        except Exception as exc:           # capture is an optimisation; the eager step is the same work
            print(f"[bench] CUDA graph capture failed on rank {rank}: {exc}", file=sys.stderr)
            run_step, graphed = step, False
        flag = torch.tensor([1 if graphed else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)      # all ranks replay graphs, or none does
        if flag.item() == 0:
            run_step, graphed = step, False
    barrier()
    with ClockSampler(local_rank) as clocks:
        t0 = time.perf_counter()
        step_ms = []
        for _ in range(args.steps):
            timing.flush_l2(device)
            barrier()                       # ranks enter the collective step together
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run_step()
            e1.record()
            e1.synchronize()
            step_ms.append(e0.elapsed_time(e1))
        barrier()
        # keep the clock sampler running for about a second; the step holds a collective, so every rank
        # must run the same number of extra steps: rank 0 decides, the others follow
        extra = torch.tensor([0], dtype=torch.int64, device=device)
        if rank == 0:
            left = 1.0 - (time.perf_counter() - t0)
            extra[0] = min(2000, max(0, int(left / max(1e-4, 1e-3 * sum(step_ms) / len(step_ms)))))
        if world > 1:
            dist.broadcast(extra, src=0)
        for _ in range(int(extra.item())):
            run_step()
        torch.cuda.synchronize(device)
    ms_per_step = sum(step_ms) / len(step_ms)
    # the decode kernel alone on this rank (roofline of the dominant kernel)
    kern = lambda: fn(q, *before, ke - kb, *after, out_dtype=torch.float16)
    kernel_ms = statistics.median(timing.time_cuda(kern, warmup=2, iters=max(args.steps, 5), device=device))
    # end to end: q from pinned host memory, output back to the host
    q_host = q.cpu().pin_memory()
    out_host = torch.empty(q.shape, dtype=torch.float16).pin_memory()
    e2e_ms = []
    for i in range(3 + args.steps):
        timing.flush_l2(device)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        o = step(q_host.to(device, non_blocking=True))
        out_host.copy_(o, non_blocking=True)
        e1.record()
        e1.synchronize()
        if i >= 3:
            e2e_ms.append(e0.elapsed_time(e1))
    e2e_mean = sum(e2e_ms) / len(e2e_ms)
    stats = torch.tensor([ms_per_step, e2e_mean, float(w["kv_bytes"]), kernel_ms], device=device, dtype=torch.float64)
    if world > 1:
        mx, sm = stats.clone(), stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms_per_step, e2e_mean, total_bytes = mx[0].item(), mx[1].item(), sm[2].item()
    else:
        total_bytes = float(w["kv_bytes"])
    if rank == 0:
        peaks = measured_peaks()
        achieved = w["kv_bytes"] / (kernel_ms * 1e-3) / 1e9
        line = dict(METRIC)
        line.update({
            "value": total_bytes / (ms_per_step * 1e-3) / 1e9, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 compute over " + fmt + " KV", "data": "synthetic",
            "config": {"workload": args.workload, "batch": 4, "h_q": 32, "h_kv": 8, "d": 128, "ctx": ctx, "page_size": page,
                       "sharding": "KV range per GPU, one all-gather of (O, LSE) per step, merge kernel on every rank",
                       "l2": "flushed between steps: 512 MB overwritten, then 256 MB read (clean cold L2)", "cuda_graph": graphed},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"], "algorithmic_bytes": w["kv_bytes"],
                         "kernel_ms": kernel_ms, "traffic": None},
            "e2e": {"value": total_bytes / (e2e_mean * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_mean,
                    "h2d_bytes_per_step": q_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": args.steps * (1 if world == 1 else 2),
            "clocks": clocks.result,
        })
        print(json.dumps(line), flush=True)
    if world > 1:
        # a captured graph holds the communicator's kernels: release it before the group goes away, and do
        # not let a stuck teardown outlive the measurement
        if graphed:
            run_step = step
            graph.reset()
            del graph, graph_out
        torch.cuda.synchronize(device)
        dist.barrier()
        import threading
        guard = threading.Timer(30.0, lambda: os._exit(0))
        guard.daemon = True
        guard.start()
        dist.destroy_process_group()
        guard.cancel()


# DRAM bytes per launch of the decode kernel from the committed ncu capture
# (profiles/paged_decode_fp16_config3.md), or None until one exists.
TRAFFIC_BYTES_PER_LAUNCH = 1303611000   # 1.299411 GB read + 4.20 MB written (mean of two captured launches)


def _use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm should use the cores this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(n, 1))


def _cpu_pass(w, max_seconds):
    """One pass of the reference CPU path over the batch (or as much of it as fits the time bound).
    Returns (seconds, kv_bytes_processed, sequences_done)."""
    from oracle import cpu_reference as R
    _use_all_host_threads()
    q = w["q"].float().cpu()
    kp, vp = w["k_pool"].cpu(), w["v_pool"].cpu()
    bt = w["block_table_host"]
    page = w["page_size"]
    h_kv, d = kp.shape[2], kp.shape[3]
    secs, done_bytes, n_done = 0.0, 0, 0
    for b, n in enumerate(w["seq_lens"]):
        k = R.gather_dense(kp, bt[b], page, n).float()      # dense fp32 KV prepared outside the timing
        v = R.gather_dense(vp, bt[b], page, n).float()
        t0 = time.perf_counter()
        R.sdpa_reference_gqa(q[b:b + 1], k, v)
        secs += time.perf_counter() - t0
        done_bytes += n * 2 * h_kv * d * 2
        n_done += 1
        if secs > max_seconds:
            break
    return secs, done_bytes, n_done


def cpu_baseline(w, bounded_s):
    _cpu_pass(w, 1.0)                                       # warm-up
    secs, nbytes, n_done = _cpu_pass(w, bounded_s)
    return {"value": nbytes / secs / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_done} of {len(w['seq_lens'])} sequences of the same batch, fp32 torch SDPA per sequence "
                      f"on dense KV (dequantise/gather outside the timing), {secs:.2f} s"}


def run_reference_long(args, dev):
    """CPU arm of the long-context workloads: the reference's GQA oracle on the dequantised keys of a
    131 072-key slice of one sequence per step (a full 1 M-key expansion does not fit host memory)."""
    from fa_bench import harness, workloads
    _use_all_host_threads()
    fmt = "e4m3" if args.workload.endswith("fp8") else "nvfp4"
    w = workloads.quantised_long_context_decode(dev, fmt=fmt, ctx=131072, batch=1)
    harness.cpu_sample(args.workload, w, 1.0)
    done, secs = 0.0, 0.0
    for _ in range(args.steps):
        d_, s_, desc = harness.cpu_sample(args.workload, w, 5.0)
        done += d_
        secs += s_
    value = done / secs / 1e9
    line = dict(METRIC)
    line.update({"impl": "reference", "value": value, "n_gpus": args.gpus, "steps": args.steps, "warmup": 1,
                 "ms_per_step": 1e3 * secs / args.steps, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                 "data": "synthetic", "config": {"workload": args.workload, "ctx": args.ctx},
                 "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port", "sample": desc},
                 "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0})
    print(json.dumps(line))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else torch.device("cpu")
    if args.workload.startswith("long_decode"):
        return run_reference_long(args, dev)
    w = build_workload(args.workload, dev, 0)
    for _ in range(max(args.warmup, 1)):
        _cpu_pass(w, 5.0)
    step_s, step_bytes = [], []
    n_done = 0
    for _ in range(args.steps):
        s, nb, n_done = _cpu_pass(w, 20.0)
        step_s.append(s)
        step_bytes.append(nb)
    value = sum(step_bytes) / sum(step_s) / 1e9
    line = dict(METRIC)
    sample = f"each step = {n_done} of {len(w['seq_lens'])} sequences of the batch on the host cores"
    line.update({
        "impl": "reference", "value": value, "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 1),
        "ms_per_step": 1e3 * sum(step_s) / len(step_s), "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": w["describe"],
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="paged_gqa_decode_fp16",
                    choices=["paged_gqa_decode_fp16", "long_decode_fp8", "long_decode_nvfp4"])
    ap.add_argument("--ctx", type=int, default=1048576, help="context length of the long-context workloads")
    ap.add_argument("--no-graph", action="store_true", help="do not replay the multi-GPU step from a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload.startswith("long_decode"):
        run_long_decode(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
