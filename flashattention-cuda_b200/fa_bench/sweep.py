"""Shape sweeps with the command line of the reference's bench/harness.py (bench/harness.py:357-397):

    python flashattention-cuda_b200/fa_bench/sweep.py --backend v8_gqa_ss --decode --seq 8192 --heads 32 \
        --gqa-group 1 4 8 --batch-sweep 1 8 64 --page-size 16

(and `--kv-lens`, `--h-kv`, `--max-ws-gb` of bench/regime.py:292-320), so that the reference's published
tables can be regenerated side by side on a B200.  Every reference
backend name is accepted (fa_kernels/dispatch.py maps it to its operator family).  One row per shape:
p50 / max milliseconds over CUDA-event samples with the L2 flushed in between, and

  prefill (default) : TFLOP/s (4 B H N^2 d, halved when causal) and the fraction of the measured bf16 peak
  --decode          : microseconds per generated token, KV GB/s and the fraction of the measured copy
                      bandwidth (K+V bytes of the H_kv heads, scales included, as bench/harness.py:296-305
                      counts them), and the speed-up over torch's scaled_dot_product_attention on the
                      same device with the KV expanded to dense fp16 (the "vs SDPA" column of the reference)

Inputs are seeded torch.randn tensors of the swept shape, as in the reference.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch  # noqa: E402

from fa_bench import timing  # noqa: E402

_MLA_DV = {576: 512, 160: 128, 96: 64}          # latent widths the MLA kernels are built for


def _peaks():
    from fa_bench import roofline
    p = roofline.measured_peaks()
    return p.hbm_gbs, p.tensor_tflops, p.source


def _time(fn, iters):
    ms = timing.time_cuda(fn, warmup=3, iters=iters)
    return statistics.median(ms), max(ms)


def _case(family, backend, B, H, G, N, d, q_len, page_size, causal, dtype, mla_engine, seed):
    """Build one shape and return (callable, sdpa callable or None, kv_bytes, flops)."""
    import fa_kernels as fk
    from fa_kernels import paged as P
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    if family == "dense":
        q, k, v = (torch.randn(B, H, N, d, device=dev, generator=g).to(dtype) for _ in range(3))
        fn = lambda: fk.attention(q, k, v, causal=causal, backend=backend)
        ref = lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)
        flops = 4.0 * B * H * N * N * d * (0.5 if causal else 1.0)
        return fn, ref, 4.0 * B * H * N * d * q.element_size(), flops
    q_off = N - q_len
    if family in ("mla", "mla_tc"):
        dv = _MLA_DV[d]
        q = torch.randn(B, H, q_len, d, device=dev, generator=g).to(torch.bfloat16)
        latent = (torch.randn(B, 1, N, d, device=dev, generator=g) * 0.1)
        lp, lm, bt, n_k, sl = P.build_paged_kv_mla(latent, page_size, seed=seed)
        if family == "mla":
            fn = lambda: fk.mla_attention(q, lp, lm, bt, page_size, n_k, dv, sl, causal=causal, q_offset=q_off, backend=backend)
        else:
            fn = lambda: fk.mla_tc_attention(q, lp, lm, bt, page_size, n_k, dv, sl, engine=mla_engine, causal=causal,
                                             q_offset=q_off, backend=backend)
        return fn, None, 1.0 * B * N * d * 0.5625, 2.0 * B * H * q_len * N * (d + dv)
    H_kv = H // G
    q = torch.randn(B, H, q_len, d, device=dev, generator=g).to(torch.float16)
    k = torch.randn(B, H_kv, N, d, device=dev, generator=g).to(torch.float16)
    v = torch.randn(B, H_kv, N, d, device=dev, generator=g).to(torch.float16)
    ke, ve = k.repeat_interleave(G, dim=1), v.repeat_interleave(G, dim=1)

    def ref():
        if q_len == 1 or not causal:
            return torch.nn.functional.scaled_dot_product_attention(q, ke, ve)
        mask = torch.ones(q_len, N, device=dev, dtype=torch.bool).tril(diagonal=q_off)
        return torch.nn.functional.scaled_dot_product_attention(q, ke, ve, attn_mask=mask)

    flops = 4.0 * B * H * q_len * N * d
    if family == "paged":
        kp, vp, bt, n_k = P.build_paged_kv(k, v, page_size, seed=seed)
        call = fk.paged_attention if backend == "v7_paged" and G == 1 else fk.gqa_attention
        fn = lambda: call(q, kp, vp, bt, page_size, n_k, causal=causal, q_offset=q_off, backend=backend)
        return fn, ref, 2.0 * B * H_kv * N * d * 2, flops
    if family == "fp8":
        kp, vp, bt, n_k, sk, sv = P.build_paged_kv_fp8(k, v, page_size, seed=seed)
        fn = lambda: fk.fp8_attention(q, kp, vp, bt, page_size, n_k, sk, sv, causal=causal, q_offset=q_off, backend=backend)
        return fn, ref, 2.0 * B * H_kv * N * d * 1, flops
    if family == "nvfp4":
        kp, km, vp, vm, bt, n_k, sk, sv = P.build_paged_kv_nvfp4(k, v, page_size, seed=seed)
        fn = lambda: fk.nvfp4_attention(q, kp, km, vp, vm, bt, page_size, n_k, sk, sv, causal=causal, q_offset=q_off,
                                        backend=backend)
        return fn, ref, 2.0 * B * H_kv * N * d * 0.5625, flops
    raise SystemExit(f"no sweep for operator family {family!r}")


def run(a):
    from fa_kernels.dispatch import _FAMILY, get_backend
    get_backend(a.backend)                       # unknown name -> KeyError, wrong GPU -> RuntimeError
    family = _FAMILY[a.backend]
    hbm, tf, src = _peaks()
    dtype = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[a.precision]
    is_mla = family in ("mla", "mla_tc")
    seqs = a.seq or ([1024, 4096, 16384] if a.decode else [512, 1024, 2048, 4096])
    dims = a.dim or ([576] if is_mla else [64, 128])
    groups = a.gqa_groups or [1]
    batches = a.batch_sweep or [a.batch]
    q_len = (a.q_len or 1) if a.decode else None
    print(f"# backend {a.backend} ({family}), peaks {src}: {hbm:.0f} GB/s, {tf:.0f} TFLOP/s bf16")
    if a.decode:
        print(f"# {'B x H x q x d / N_k':>26} | ms p50 / max     | us/token | KV GB/s | of copy peak | vs SDPA")
    else:
        print(f"# {'B x H x N x d':>26} | ms p50 / max     | TFLOP/s | of bf16 peak | vs SDPA")
    rows = []
    head_sets = [(G * hk, G) for hk in a.h_kvs for G in groups] if a.h_kvs else [(a.heads, G) for G in groups]
    for B in batches:
        for heads, G in head_sets:
            if heads % G:
                raise SystemExit(f"--heads {heads} is not divisible by --gqa-group {G}")
            a.heads = heads
            for d in dims:
                for N in seqs:
                    if 2.0 * B * (heads // G) * N * d * 2 > a.max_ws_gb * 1e9 and not is_mla and family != "dense":
                        print(f"  {f'{B}x{heads}x.x{d}/{N}':>26} | skipped: dense K+V above --max-ws-gb")
                        continue
                    ql = q_len if a.decode else N
                    fn, ref, kv_bytes, flops = _case(family, a.backend, B, a.heads, G, N, d, ql, a.page_size, a.causal, dtype,
                                                     a.mla_engine, seed=B * 131 + N)
                    p50, mx = _time(fn, a.iters)
                    vs = float("nan")
                    if ref is not None:
                        try:
                            vs = _time(ref, max(3, a.iters // 3))[0] / p50
                        except RuntimeError:                # SDPA ran out of memory at this shape
                            torch.cuda.empty_cache()
                    label = f"{B}x{a.heads}x{ql}x{d}" + (f"/{N}" if a.decode else "") + (f" G{G}" if G > 1 else "")
                    row = {"shape": label, "ms_p50": p50, "ms_max": mx, "vs_sdpa": vs}
                    if a.decode:
                        gbs = kv_bytes / (p50 * 1e-3) / 1e9
                        row.update(us_per_token=p50 * 1e3 / (B * ql), kv_gbs=gbs, frac_of_copy_peak=gbs / hbm)
                        print(f"  {label:>26} | {p50:7.3f} / {mx:7.3f} | {row['us_per_token']:8.2f} | {gbs:7.0f} | "
                              f"{100 * gbs / hbm:11.1f}% | {vs:6.2f}x")
                    else:
                        tfs = flops / (p50 * 1e-3) / 1e12
                        row.update(tflops=tfs, frac_of_bf16_peak=tfs / tf)
                        print(f"  {label:>26} | {p50:7.3f} / {mx:7.3f} | {tfs:7.1f} | {100 * tfs / tf:11.1f}% | {vs:6.2f}x")
                    rows.append(row)
                    torch.cuda.empty_cache()
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)
    return rows


def build_parser():
    p = argparse.ArgumentParser(description="Shape sweeps with the reference harness's command line.")
    p.add_argument("--backend", default="v8_gqa_ss")
    p.add_argument("--precision", default="fp16", choices=["fp32", "fp16", "bf16"])
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--batch-sweep", type=int, nargs="+", default=None, dest="batch_sweep")
    p.add_argument("--page-size", type=int, default=64, dest="page_size")
    p.add_argument("--heads", type=int, default=8)
    p.add_argument("--causal", action="store_true")
    p.add_argument("--seq", "--kv-lens", type=int, nargs="+", default=None, dest="seq",
                   help="sequence lengths (KV lengths with --decode); --kv-lens is the spelling of bench/regime.py")
    p.add_argument("--h-kv", type=int, nargs="+", default=None, dest="h_kvs",
                   help="bench/regime.py style: sweep the KV heads, H_q = gqa-group x H_kv (overrides --heads)")
    p.add_argument("--max-ws-gb", type=float, default=16.0, dest="max_ws_gb",
                   help="skip shapes whose dense fp16 K+V exceed this many GB (bench/regime.py:312)")
    p.add_argument("--dim", type=int, nargs="+", default=None)
    p.add_argument("--decode", action="store_true")
    p.add_argument("--q-len", type=int, default=None, dest="q_len")
    p.add_argument("--mla-engine", default="fp8", choices=["fp8", "nvfp4"], dest="mla_engine")
    p.add_argument("--gqa-group", type=int, nargs="+", default=None, dest="gqa_groups")
    p.add_argument("--iters", type=int, default=15)
    p.add_argument("--json", default=None, help="also write the rows to this file")
    return p


def main():
    a = build_parser().parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device; the sweep runs on the GPU")
    run(a)


if __name__ == "__main__":
    main()
