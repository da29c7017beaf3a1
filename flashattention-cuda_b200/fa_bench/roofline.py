"""Three-resource lower bound for the attention workloads, on this machine's measured peaks.

The method of the reference's `roofline/model.py:53-230`: count the work of a launch on the three
resources attention can run out of (tensor-core FLOPs of the two matrix products, HBM bytes, MUFU
exponentials), divide each by its peak rate, and the largest quotient is the time no kernel can beat; the
resource that owns it is the limiter.  The reference evaluates this on data-sheet constants
(`roofline/archs.py:108-124`, tagged speculative for B200); here the rates are the copy bandwidth and
bf16 GEMM throughput measured on the pool's own B200s (MEASURED_PEAKS.json at the repository root, written
by the test driver), with the data-sheet figures as the documented fallback.

The work counts are the single source of the `algorithmic_bytes` / FLOP figures that bench.py and
fa_bench/harness.py divide by the measured kernel time.

    python flashattention-cuda_b200/fa_bench/roofline.py        # the five benchmark configurations
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# bytes per stored element of a KV / latent format; "nvfp4" counts the E4M3 micro-scale of every 16
# elements (4.5 bits per element, reference roofline/model.py:27-30)
BYTES_PER_ELEM = {"f32": 4.0, "f16": 2.0, "bf16": 2.0, "e4m3": 1.0, "nvfp4": 0.5625}

SM_COUNT = 148
MUFU_PER_SM_PER_CLK = 16          # ex2.approx.f32 results per SM per cycle


@dataclass(frozen=True)
class Peaks:
    hbm_gbs: float                # GB/s
    tensor_tflops: float          # dense bf16 / fp16 TFLOP/s, a kernel timed alone (burst)
    tensor_tflops_sustained: float
    exp_per_s: float              # MUFU exponentials per second
    source: str                   # "measured" | "fallback" | "nominal"


def measured_peaks(path: str | None = None) -> Peaks:
    """MEASURED_PEAKS.json when present ("measured"), else the earlier measurement of this pool that the
    profiling notes give as the fallback (6.65 TB/s, 1.59 PFLOP/s burst, ~1.4 sustained)."""
    path = path or os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        mhz = float(d.get("sm_max_mhz", 1965.0))
        return Peaks(float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                     SM_COUNT * MUFU_PER_SM_PER_CLK * mhz * 1e6, "measured")
    return Peaks(6650.0, 1590.0, 1400.0, SM_COUNT * MUFU_PER_SM_PER_CLK * 1965e6, "fallback")


def nominal_peaks() -> Peaks:
    """Data-sheet B200: 8 TB/s, 2.25 PFLOP/s dense fp16 (the reference's `B200` entry, archs.py:108-124)."""
    return Peaks(8000.0, 2250.0, 2250.0, SM_COUNT * MUFU_PER_SM_PER_CLK * 1965e6, "nominal")


@dataclass(frozen=True)
class Work:
    """Algorithmic work of one launch."""
    flops: float                  # tensor-core FLOPs (both matrix products)
    kv_bytes: float               # the streamed operand alone (KV cache / latent / K and V), what "% of HBM" counts
    total_bytes: float            # kv_bytes + queries + outputs (+ block table)
    exps: float                   # softmax exponentials
    bound: str                    # "hbm" | "tensor": which roofline the workload is graded on

    @property
    def intensity(self) -> float:
        return self.flops / self.total_bytes


def dense_attention(B: int, H: int, N_q: int, N_k: int, d: int, *, causal: bool, elem: str = "f16") -> Work:
    """Fused dense attention (reference model.py:137-142, 197-206 with S kept on chip).  Causal square
    attention computes the lower triangle only: 2 B H d N (N + 1) FLOPs; the reference counts the full
    4 B H N^2 d, reported by `dense_attention_full_flops`."""
    b = BYTES_PER_ELEM[elem]
    pairs = N_q * N_k
    if causal:
        n = min(N_q, N_k)
        pairs = n * (n + 1) // 2 + max(N_q - n, 0) * N_k
    flops = 4.0 * B * H * d * pairs
    io = (2.0 * B * H * N_k * d + 2.0 * B * H * N_q * d) * b
    return Work(flops, 2.0 * B * H * N_k * d * b, io, float(B * H * pairs), "tensor")


def dense_attention_full_flops(B: int, H: int, N_q: int, N_k: int, d: int) -> float:
    return 4.0 * B * H * N_q * N_k * d


def paged_decode(tokens: int, *, H_q: int, H_kv: int, d: int, kv_format: str = "f16", per_token_scales: bool = False,
                 B: int = 1, N_q: int = 1, table_entries: int = 0) -> Work:
    """Paged GQA decode over `tokens` = sum of the context lengths: every token's K and V rows are read
    once for the whole query group (reference model.py:188-199 with KV bytes / G), plus one fp32 scale per
    token per head and tensor for per-token FP8."""
    row = d * BYTES_PER_ELEM[kv_format] + (4.0 if per_token_scales else 0.0)
    kv = 2.0 * H_kv * tokens * row
    io = 2.0 * B * H_q * N_q * d * 2.0 + 4.0 * table_entries
    return Work(4.0 * H_q * d * tokens * N_q, kv, kv + io, float(H_q * tokens * N_q), "hbm")


def mla_decode(tokens: int, *, h_q: int, dqk: int = 576, dv: int = 512, latent_format: str = "bf16",
               per_token_scales: bool = False, B: int = 1, N_q: int = 1) -> Work:
    """MLA latent decode: one latent row per token serves as key (dqk dims) and value (dv dims) for all
    h_q heads (reference model.py:107-116): FLOPs = 2 h_q (dqk + dv) per token, bytes = dqk x width."""
    row = dqk * BYTES_PER_ELEM[latent_format] + (4.0 if per_token_scales else 0.0)
    kv = tokens * row
    io = B * h_q * N_q * (dqk + dv) * 2.0
    return Work(2.0 * h_q * (dqk + dv) * tokens * N_q, kv, kv + io, float(h_q * tokens * N_q), "tensor")


def lower_bound(work: Work, peaks: Peaks) -> dict:
    """Times of the three resources if each were alone, the limiter and the bound (seconds)."""
    t = {"mma": work.flops / (peaks.tensor_tflops * 1e12), "hbm": work.total_bytes / (peaks.hbm_gbs * 1e9),
         "mufu": work.exps / peaks.exp_per_s}
    limiter = max(t, key=t.get)
    return {"t_mma": t["mma"], "t_hbm": t["hbm"], "t_mufu": t["mufu"], "limiter": limiter, "seconds": t[limiter],
            "arithmetic_intensity": work.intensity, "ridge": peaks.tensor_tflops * 1e12 / (peaks.hbm_gbs * 1e9),
            "peak_source": peaks.source}


def achieved(work: Work, seconds: float, peaks: Peaks) -> dict:
    """The `roofline` object of a bench line for a launch that took `seconds`."""
    if work.bound == "hbm":
        a, peak, unit, alg = work.kv_bytes / seconds / 1e9, peaks.hbm_gbs, "GB/s", work.kv_bytes
    else:
        a, peak, unit, alg = work.flops / seconds / 1e12, peaks.tensor_tflops, "TFLOP/s", work.flops
    out = {"bound": work.bound, "achieved": a, "peak": peak, "unit": unit, "frac": a / peak, "peak_source": peaks.source,
           "algorithmic_work": alg, "kernel_ms": seconds * 1e3, "lower_bound_ms": lower_bound(work, peaks)["seconds"] * 1e3,
           "limiter": lower_bound(work, peaks)["limiter"]}
    if work.bound == "hbm":
        out["frac_of_nominal_8TBs"] = a / 8000.0
    else:
        out["frac_of_nominal_2250TF"] = a / 2250.0
    return out


# expected token counts of the benchmark configurations (uniform context lengths)
BENCH_CONFIGS = {
    "causal_prefill_fp16": lambda: dense_attention(4, 32, 4096, 4096, 128, causal=True),
    "paged_gqa_decode_fp16": lambda: paged_decode(64 * 4608, H_q=32, H_kv=8, d=128, B=64),
    "long_decode_fp8": lambda: paged_decode(4 * 1048576, H_q=32, H_kv=8, d=128, kv_format="e4m3", per_token_scales=True, B=4),
    "long_decode_nvfp4": lambda: paged_decode(4 * 1048576, H_q=32, H_kv=8, d=128, kv_format="nvfp4", B=4),
    "mla_decode_bf16": lambda: mla_decode(128 * 18432, h_q=128, B=128),
    "mla_decode_fp8": lambda: mla_decode(128 * 18432, h_q=128, latent_format="e4m3", per_token_scales=True, B=128),
}


def main():
    for peaks in (measured_peaks(), nominal_peaks()):
        print(f"# peaks: {peaks.source}: {peaks.hbm_gbs:.0f} GB/s, {peaks.tensor_tflops:.0f} TFLOP/s, {peaks.exp_per_s / 1e12:.2f} Texp/s")
        for name, make in BENCH_CONFIGS.items():
            w = make()
            lb = lower_bound(w, peaks)
            print(f"{name:24s} flops {w.flops:.4g}  bytes {w.total_bytes:.4g}  AI {w.intensity:7.1f} (ridge {lb['ridge']:.0f})  "
                  f"mma {lb['t_mma'] * 1e3:.3f} ms  hbm {lb['t_hbm'] * 1e3:.3f} ms  mufu {lb['t_mufu'] * 1e3:.3f} ms  -> {lb['limiter']}")


if __name__ == "__main__":
    main()
