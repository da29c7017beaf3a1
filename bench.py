"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one pass of the hot path over one batch of seeded synthetic input.  The headline workload is the
paged GQA decode configuration (fp16 KV, batch 64, 32 query / 8 KV heads, d=128, context lengths uniform
in [1024, 8192], 16-token pages, shuffled block table); the metric is the KV bytes streamed per second.
Rank 0 prints one JSON line.

* One GPU: the line also carries a `workloads` array with one entry per other benchmark configuration at
  full size (causal prefill, MLA decode with a bf16 and an FP8 latent, FP8 and NVFP4 long-context decode),
  each with its own median time, algorithmic work and roofline fraction.
* N GPUs (torchrun): the same 64-sequence batch is dealt to the ranks by token count (strong scaling, no
  collective on the data path); each rank times on its own device with CUDA events and the slowest rank
  defines the step.  The line adds `per_rank_step_ms`, the weak-scaling figure (one whole batch per rank),
  the MLA batch dealt the same way, and a `kv_range` entry: the FP8 long-context decode with every
  sequence's keys cut into one range per rank, one NCCL all-gather of (O, LSE) and the merge kernel.

`--impl reference` times the reference project's CPU implementation of the same path (torch SDPA through
the wrappers of its fa_kernels/reference.py, restated in oracle/cpu_reference.py) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(REPO, "flashattention-cuda_b200"))
sys.path.insert(0, REPO)

import torch  # noqa: E402

METRIC = {"metric": "decode_kv_gbs", "unit": "GB/s", "higher_is_better": True}
HEADLINE = "paged_gqa_decode_fp16"
METHOD = {
    "l2": "flushed before every timed launch, outside the event window: 512 MB overwritten, then 256 MB read so "
          "that the cold L2 holds no dirty lines",
    "timing": "CUDA events on the launching stream around each step; a ~0.3 ms spin kernel sits between the flush "
              "and the start event so that the host has enqueued the step before the window opens; per rank the "
              "median over the steps, over ranks the maximum",
}


class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
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


def dist_env():
    return int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


def init_dist(args):
    import torch.distributed as dist
    world, rank, local_rank = dist_env()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    return world, rank, local_rank, device


def teardown_dist(world):
    """Leave the process group; a teardown that does not return is reported as a failure, not hidden."""
    import torch.distributed as dist
    if world <= 1:
        return
    torch.cuda.synchronize()
    dist.barrier()

    def stuck():
        print("[bench] destroy_process_group did not return within 60 s", file=sys.stderr, flush=True)
        os._exit(3)
    guard = threading.Timer(60.0, stuck)
    guard.daemon = True
    guard.start()
    dist.destroy_process_group()
    guard.cancel()


def gather_lists(values, world, device):
    """Every rank's list of floats (equal lengths) -> list of lists on every rank."""
    import torch.distributed as dist
    t = torch.tensor(values, dtype=torch.float64, device=device)
    if world == 1:
        return [t.tolist()]
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [o.tolist() for o in out]


def headline_lens():
    """Context lengths of the 64-sequence batch (seed 2, CPU generator: the same on every rank)."""
    g = torch.Generator(device="cpu").manual_seed(2)
    return torch.randint(1024, 8193, (64,), generator=g).tolist()


# --------------------------------------------------------------------------------------------------
# the headline workload: paged GQA decode, fp16, the 64-sequence batch dealt over the ranks
# --------------------------------------------------------------------------------------------------
def timed_steps(step, steps, warmup, device, barrier):
    from fa_bench import timing
    for _ in range(max(warmup, 3)):
        timing.flush_l2(device)
        step()
    barrier()
    ms = timing.time_cuda(step, warmup=0, iters=steps, device=device)
    barrier()
    return ms


def run_ours(args):
    import torch.distributed as dist
    from fa_bench import harness, roofline, timing
    from fa_kernels import HostDecodeStep, _lib, check_status, gqa_attention
    from fa_kernels.distributed import shard_batch_by_length

    world, rank, local_rank, device = init_dist(args)
    _lib.load()                                     # no library, no benchmark

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    lens_all = headline_lens()
    owned = shard_batch_by_length(lens_all, world)[rank]
    my_lens = [lens_all[i] for i in owned]
    case = harness.build(HEADLINE, device, seq_lens=my_lens, data_seed=2 + 1000 * rank)
    w, step = case["w"], case["step"]
    page = w["page_size"]

    with ClockSampler(local_rank) as clocks:
        t_wall0 = time.perf_counter()
        step_ms = timed_steps(step, args.steps, args.warmup, device, barrier)
        # keep the GPU busy long enough for the 200 ms clock sampler to see it under load
        while time.perf_counter() - t_wall0 < 1.2:
            step()
        torch.cuda.synchronize(device)
    check_status(device)

    # ---- end to end through the C ABI with host buffers: one fa_paged_decode_host call per step --------
    # q, block table and the sequence lengths come from pinned host memory, the plan is rebuilt for the step's
    # lengths (a serving step has new lengths), the output lands in pinned host memory; the KV cache is
    # resident device state.
    q_host = w["q"].cpu().pin_memory()
    bt_host = w["block_table_host"].pin_memory()
    lens_host = torch.tensor(my_lens, dtype=torch.int32).pin_memory()
    out_host = torch.empty(w["q"].shape, dtype=torch.float16).pin_memory()
    B_, Hq_, Nq_, d_ = w["q"].shape
    host_step = HostDecodeStep(w["k_pool"], w["v_pool"], page, B_, Hq_, Nq_, d_, bt_host.shape[1], out_dtype=torch.float16)
    # The host's own work (argument checks, planner) belongs to this number, so the window opens on an idle,
    # synchronised GPU and nothing hides the host time.
    e2e_ms = []
    for i in range(3 + args.steps):
        timing.flush_l2(device)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        host_step(q_host, bt_host, lens_host, out_host)
        e1.record()
        e1.synchronize()
        if i >= 3:
            e2e_ms.append(e0.elapsed_time(e1))
    barrier()
    check = gqa_attention(w["q"], w["k_pool"], w["v_pool"], w["block_table"], page, my_lens, out_dtype=torch.float16)
    torch.cuda.synchronize(device)
    assert torch.equal(check.cpu(), out_host), "host-buffer step and device-tensor API disagree"
    check_status(device)
    from fa_kernels import _decode
    n_items = _decode.plan(tuple(my_lens), max(my_lens), B_, w["k_pool"].shape[2], (Hq_ // w["k_pool"].shape[2]) * Nq_, page, device, 0, 2)[1]
    h2d = q_host.numel() * 2 + bt_host.numel() * 4 + n_items * 32        # lengths are read by the host planner
    d2h = out_host.numel() * 2

    # ---- reduce over ranks ------------------------------------------------------------------------------
    per_rank_steps = gather_lists(step_ms, world, device)
    per_rank_e2e = gather_lists(e2e_ms, world, device)
    per_rank_meta = gather_lists([float(w["kv_bytes"]), float(w["tokens"]), float(len(my_lens)), float(h2d), float(d2h)], world, device)
    per_rank_ms = [statistics.median(x) for x in per_rank_steps]
    ms_per_step = max(per_rank_ms)
    e2e_ms_step = max(statistics.median(x) for x in per_rank_e2e)
    total_kv_bytes = sum(m[0] for m in per_rank_meta)

    extra = {}
    if world > 1:
        extra["weak_replicas"] = weak_replicas(args, world, rank, device, barrier)
        extra["mla_batch_sharded"] = mla_batch_sharded(args, world, rank, device, barrier)
        extra["kv_range"] = long_decode(args, "long_decode_fp8", world, rank, local_rank, device, quiet=True)
    else:
        del host_step, case, w, step, check
        torch.cuda.empty_cache()
        extra["workloads"] = other_workloads(args, device, local_rank)

    if rank == 0:
        peaks = roofline.measured_peaks()
        slow = per_rank_ms.index(ms_per_step)
        work0 = roofline.paged_decode(int(per_rank_meta[slow][1]), H_q=32, H_kv=8, d=128, B=int(per_rank_meta[slow][2]))
        roof = roofline.achieved(work0, ms_per_step * 1e-3, peaks)      # the slowest rank's launch
        full = roofline.paged_decode(sum(lens_all), H_q=32, H_kv=8, d=128, B=64)
        traffic, src = harness.captured_traffic(HEADLINE, work0)
        roof["traffic"], roof["traffic_source"] = traffic, src
        roof["note"] = ("every timed step is exactly one launch of paged_decode_kernel; kernel_ms is the median CUDA-event "
                        "duration of that launch on the slowest rank, algorithmic_work that rank's KV bytes")
        line = dict(METRIC)
        line.update({
            "value": total_kv_bytes / (ms_per_step * 1e-3) / 1e9,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": headline_config(lens_all),
            "method": dict(METHOD, sharding="the 64 sequences are dealt to the ranks longest first by token count; "
                                            "no collective on the data path"),
            "step_ms": dict(timing.summary(per_rank_steps[slow]), rank=slow),
            "per_rank_ms": per_rank_ms,
            "per_rank_step_ms": per_rank_steps,
            "per_rank_kv_tokens": [int(m[1]) for m in per_rank_meta],
            "roofline": roof,
            "lower_bound_ms_whole_batch_one_gpu": roofline.lower_bound(full, peaks)["seconds"] * 1e3,
            "e2e": {"value": total_kv_bytes / (e2e_ms_step * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms_step,
                    "h2d_bytes_per_step": int(sum(m[3] for m in per_rank_meta)), "d2h_bytes_per_step": int(sum(m[4] for m in per_rank_meta)),
                    "note": "one fa_paged_decode_host call per step and rank (fa_kernels.HostDecodeStep): q, block table and the "
                            "step's split plan copied from pinned host memory, output copied back to pinned host memory; "
                            "the KV cache is resident device state"},
            "gpu_launches": args.steps,
            "clocks": clocks.result,
        })
        line.update(extra)
        if world == 1:
            line["cpu_baseline"] = cpu_baseline_headline(bounded_s=20.0)
        print(json.dumps(line), flush=True)
    teardown_dist(world)


def headline_config(lens_all):
    return {"workload": HEADLINE, "batch": 64, "h_q": 32, "h_kv": 8, "d": 128, "page_size": 16,
            "ctx": "uniform[1024,8192] seed 2", "kv_tokens": sum(lens_all)}


def weak_replicas(args, world, rank, device, barrier):
    """The weak-scaling figure: every rank owns a whole 64-sequence batch (same lengths, its own values)."""
    from fa_bench import harness
    case = harness.build(HEADLINE, device, data_seed=2 + 1000 * rank)
    ms = timed_steps(case["step"], args.steps, 3, device, barrier)
    per_rank = [statistics.median(x) for x in gather_lists(ms, world, device)]
    total = case["w"]["kv_bytes"] * world
    del case
    torch.cuda.empty_cache()
    return {"scaling": "weak", "batch_per_gpu": 64, "ms_per_step": max(per_rank), "per_rank_ms": per_rank,
            "value": total / (max(per_rank) * 1e-3) / 1e9, "unit": "GB/s"}


def mla_batch_sharded(args, world, rank, device, barrier):
    """MLA latent decode (bf16 latent, 128 sequences, context uniform in [4096, 32768]) with the sequences
    dealt to the ranks by token count; no collective on the data path."""
    from fa_bench import harness
    from fa_kernels.distributed import shard_batch_by_length
    g = torch.Generator(device="cpu").manual_seed(5)
    lens_all = torch.randint(4096, 32769, (128,), generator=g).tolist()
    mine = [lens_all[i] for i in shard_batch_by_length(lens_all, world)[rank]]
    case = harness.build("mla_decode_bf16", device, seq_lens=mine)
    ms = timed_steps(case["step"], max(5, args.steps // 2), 3, device, barrier)
    per_rank = [statistics.median(x) for x in gather_lists(ms, world, device)]
    flops = 2 * 128 * (576 + 512) * sum(lens_all)
    del case
    torch.cuda.empty_cache()
    return {"workload": "mla_decode_bf16", "scaling": "strong", "ms_per_step": max(per_rank), "per_rank_ms": per_rank,
            "value": flops / (max(per_rank) * 1e-3) / 1e12, "unit": "TFLOP/s"}


def other_workloads(args, device, local_rank):
    """One entry per remaining benchmark configuration at full size (one GPU)."""
    from fa_bench import harness
    from fa_kernels import check_status
    rows = []
    for name in ("causal_prefill_fp16", "mla_decode_bf16", "mla_decode_fp8", "long_decode_fp8", "long_decode_nvfp4"):
        case = harness.build(name, device)
        torch.cuda.synchronize(device)
        with ClockSampler(local_rank) as clocks:
            row = harness.measure(name, device, iters=max(args.steps, 10), warmup=max(args.warmup, 3), hold_seconds=1.0, case=case)
        check_status(device)
        row["clocks"] = clocks.result
        row["cpu_baseline"] = cpu_sample(name, case["w"], 4.0)
        rows.append(row)
        del case
        torch.cuda.empty_cache()
    return rows


# --------------------------------------------------------------------------------------------------
# KV-range sharded long-context decode (strong scaling with one all-gather per step)
# --------------------------------------------------------------------------------------------------
def long_decode(args, workload, world, rank, local_rank, device, quiet=False):
    """Quantised-KV long-context decode (B=4, context 1 048 576, page 64), sharded by KV range: rank r owns the
    keys of logical pages [r*P/N, (r+1)*P/N) of every sequence in its own pool; one step = local decode +
    one NCCL all-gather of (O, LSE) + merge on every rank.  Strong scaling: the context is fixed."""
    import torch.distributed as dist
    from fa_bench import roofline, timing, workloads
    from fa_kernels import check_status, fp8_attention, nvfp4_attention
    from fa_kernels.distributed import kv_range_decode, kv_range_shards

    fmt = "e4m3" if workload.endswith("fp8") else "nvfp4"
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
    run_step, graphed, graph = step, False, None
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
            run_step, graphed, graph = step, False, None
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
            timing.hold_gpu(device)
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
            extra[0] = min(2000, max(0, int(left / max(1e-4, 1e-3 * statistics.median(step_ms)))))
        if world > 1:
            dist.broadcast(extra, src=0)
        for _ in range(int(extra.item())):
            run_step()
        torch.cuda.synchronize(device)
    # the decode kernel alone on this rank (roofline of the dominant kernel)
    kern = lambda: fn(q, *before, ke - kb, *after, out_dtype=torch.float16)
    kernel_ms = statistics.median(timing.time_cuda(kern, warmup=2, iters=max(args.steps, 5), device=device))
    check_status(device)
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
    per_rank_steps = gather_lists(step_ms, world, device)
    per_rank_ms = [statistics.median(x) for x in per_rank_steps]
    ms_per_step = max(per_rank_ms)
    e2e = max(statistics.median(x) for x in gather_lists(e2e_ms, world, device))
    per_rank_kernel = [x[0] for x in gather_lists([kernel_ms], world, device)]
    total_bytes = sum(x[0] for x in gather_lists([float(w["kv_bytes"])], world, device))
    if graphed:
        # a captured graph holds the communicator's kernels: release it before the group goes away
        run_step = step
        graph.reset()
        del graph, graph_out
        torch.cuda.synchronize(device)
    result = None
    if rank == 0:
        peaks = roofline.measured_peaks()
        work = roofline.paged_decode(4 * (ke - kb), H_q=32, H_kv=8, d=128, kv_format=fmt, per_token_scales=(fmt == "e4m3"), B=4)
        roof = roofline.achieved(work, per_rank_kernel[0] * 1e-3, peaks)
        roof["traffic"] = None
        result = {
            "value": total_bytes / (ms_per_step * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "ms_per_step": ms_per_step, "per_rank_ms": per_rank_ms, "scaling": "strong",
            "decode_kernel_ms": max(per_rank_kernel), "exchange_ms": ms_per_step - max(per_rank_kernel),
            "exchange": "one all_gather_into_tensor of [B*H_q*(D+1)] floats per rank (NCCL) + merge_partials_kernel on every rank"
                        if world > 1 else "none (one GPU holds the whole range)",
            "config": {"workload": workload, "batch": 4, "h_q": 32, "h_kv": 8, "d": 128, "ctx": ctx, "page_size": page},
            "cuda_graph": graphed, "roofline": roof,
            "e2e": {"value": total_bytes / (e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e,
                    "h2d_bytes_per_step": q_host.numel() * 2 * world, "d2h_bytes_per_step": out_host.numel() * 2 * world},
            "clocks": clocks.result,
        }
    del w, before, after
    torch.cuda.empty_cache()
    if quiet or rank != 0:
        return result
    line = dict(METRIC)
    line.update({"warmup": max(args.warmup, 3), "vs_baseline": None, "dtype": "f16 compute over " + fmt + " KV", "data": "synthetic",
                 "method": dict(METHOD, sharding="KV range per GPU, one all-gather of (O, LSE) per step, merge kernel on every rank"),
                 "gpu_launches": args.steps * (1 if world == 1 else 2)})
    line.update(result)
    print(json.dumps(line), flush=True)
    return result


def run_long_decode(args):
    from fa_kernels import _lib
    world, rank, local_rank, device = init_dist(args)
    _lib.load()
    long_decode(args, args.workload, world, rank, local_rank, device)
    teardown_dist(world)


# --------------------------------------------------------------------------------------------------
# CPU legs: the reference's own CPU implementation of the path, timed on this machine's host cores.
# (The only place where the product side of this file touches oracle/.)
# --------------------------------------------------------------------------------------------------
def _use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm should use the cores this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(n, 1))


def _cpu_pass(w, max_seconds):
    """One pass of the reference CPU path over the decode batch (or as much of it as fits the time bound).
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


def cpu_baseline_headline(bounded_s, device=None):
    from fa_bench import workloads
    dev = device or (torch.device("cuda", dist_env()[2]) if torch.cuda.is_available() else torch.device("cpu"))
    w = workloads.paged_gqa_decode(dev, seed=2, data_seed=2)
    _cpu_pass(w, 1.0)                                       # warm-up
    secs, nbytes, n_done = _cpu_pass(w, bounded_s)
    return {"value": nbytes / secs / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_done} of {len(w['seq_lens'])} sequences of the same batch, fp32 torch SDPA per sequence "
                      f"on dense KV (dequantise/gather outside the timing), {secs:.2f} s"}


def cpu_sample(name, w, seconds):
    """The reference CPU path on a bounded sample of one of the other workloads -> cpu_baseline object."""
    from fa_kernels import paged as P
    from oracle import cpu_reference as R
    _use_all_host_threads()
    t_used, reps = 0.0, 0
    if name.startswith("long_decode"):
        n = 131072                                           # one sequence, 128 Ki keys, scaled linearly
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
        while t_used < seconds:
            t0 = time.perf_counter()
            R.sdpa_reference_gqa(q, k, v)
            t_used += time.perf_counter() - t0
            reps += 1
        done, unit, desc = reps * n * per_tok / 1e9, "GB/s", f"{reps} passes over the first 131072 keys of sequence 0 (dequantised outside the timing)"
    elif name == "causal_prefill_fp16":
        q, k, v = (w[x][:1, :2].float().cpu() for x in ("q", "k", "v"))
        while t_used < seconds:
            t0 = time.perf_counter()
            R.sdpa_reference(q, k, v, causal=True)
            t_used += time.perf_counter() - t0
            reps += 1
        n, d = q.shape[2], q.shape[3]
        done, unit, desc = reps * 2 * 2 * d * n * (n + 1) / 1e12, "TFLOP/s", f"{reps} passes over 2 of {w['q'].shape[0] * w['q'].shape[1]} heads, fp32 SDPA"
    elif name.startswith("mla_decode"):
        n = min(w["seq_lens"][0], 8192)
        bt = w["block_table"][:1].contiguous()
        lat = P.paged_gather(w["l_pool"], bt, w["page_size"], n)
        if name.endswith("fp8"):
            lat = P.dequantize_fp8_e4m3(lat, P.paged_gather(w["scale_l"].unsqueeze(-1), bt, w["page_size"], n)[..., 0])
        lat, q = lat.float().cpu(), w["q"][:1].float().cpu()
        while t_used < seconds:
            t0 = time.perf_counter()
            R.sdpa_reference_mla_dequantised(q, lat, w["kv_lora_rank"])
            t_used += time.perf_counter() - t0
            reps += 1
        done, unit, desc = reps * 2 * q.shape[1] * (q.shape[3] + w["kv_lora_rank"]) * n / 1e12, "TFLOP/s", f"{reps} passes over the first {n} keys of sequence 0"
    else:
        raise ValueError(name)
    return {"value": done / t_used, "unit": unit, "cores": torch.get_num_threads(), "kind": "port", "sample": desc + f", {t_used:.1f} s"}


def run_reference(args):
    """The reference arm: its CPU path on the host cores.  Rank 0 alone works; under strong scaling the job
    at every N is the same 64-sequence batch, so the CPU arm does the same total work at every N."""
    world, rank, local_rank = dist_env()
    if rank != 0:
        return
    dev = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    from fa_bench import workloads
    if args.workload.startswith("long_decode"):
        fmt = "e4m3" if args.workload.endswith("fp8") else "nvfp4"
        w = workloads.quantised_long_context_decode(dev, fmt=fmt, ctx=131072, batch=1)
        cpu_sample(args.workload, w, 1.0)
        vals = [cpu_sample(args.workload, w, 5.0) for _ in range(args.steps)]
        value = statistics.mean(v["value"] for v in vals)
        config, ms, sample = {"workload": args.workload, "batch": 4, "h_q": 32, "h_kv": 8, "d": 128, "ctx": args.ctx, "page_size": 64}, 5e3, vals[-1]["sample"]
    else:
        w = workloads.paged_gqa_decode(dev, seed=2, data_seed=2)
        for _ in range(max(args.warmup, 1)):
            _cpu_pass(w, 5.0)
        step_s, step_bytes, n_done = [], [], 0
        for _ in range(args.steps):
            s, nb, n_done = _cpu_pass(w, 20.0)
            step_s.append(s)
            step_bytes.append(nb)
        value = sum(step_bytes) / sum(step_s) / 1e9
        config, ms = headline_config(w["seq_lens"]), 1e3 * sum(step_s) / len(step_s)
        sample = f"each step = {n_done} of {len(w['seq_lens'])} sequences of the batch on the host cores"
    line = dict(METRIC)
    line.update({
        "impl": "reference", "value": value, "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 1),
        "ms_per_step": ms, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=HEADLINE, choices=[HEADLINE, "long_decode_fp8", "long_decode_nvfp4"])
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
