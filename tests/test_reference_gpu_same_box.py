"""This library's kernels against the reference project's own CUDA kernels on the same GPU and the same tensors.

The reference's kernel versions of the hot path (v5_wmma, v8_gqa_ss, v9_fp8, v10_nvfp4, v11_mla) are built for
sm_100a by oracle/build_reference_gpu.py into oracle/_ref/ (from the reference's sources where they lie; the
shared objects are not part of the repository).  Where they are present, each test runs the reference module's
`forward` (the call of the reference's fa_kernels wrappers, e.g. fa_kernels/paged.py:232-234, 258-260, 282-284,
337-340) and this library's operator on identical device tensors, requires the two outputs to agree within the
path's tolerance, and prints one `SAME_BOX` JSON row with both CUDA-event medians (L2 flushed before every
launch).  Shapes follow the benchmark configurations with one length for every sequence and per-tensor FP8
scales, which is what the reference's interface takes.  Without oracle/_ref the tests are skipped.

    python -m pytest tests/test_reference_gpu_same_box.py -m gpu -q -s
"""

from __future__ import annotations

import importlib.machinery
import importlib.util
import json
import os

import pytest
import torch

from conftest import PKG_DIR  # noqa: F401  (puts the package on sys.path)

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _reference_module(version):
    path = os.path.join(REF_DIR, version, f"fa_{version}.so")
    if not os.path.exists(path):
        pytest.skip(f"{path} not built (python oracle/build_reference_gpu.py)")
    name = f"fa_{version}"
    loader = importlib.machinery.ExtensionFileLoader(name, path)
    spec = importlib.util.spec_from_file_location(name, path, loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


def _time_both(name, ours, theirs, config, iters=7):
    from fa_bench import timing
    dev = torch.device("cuda:0")
    t_ours = timing.summary(timing.time_cuda(ours, warmup=2, iters=iters, device=dev))["p50"]
    t_ref = timing.summary(timing.time_cuda(theirs, warmup=2, iters=iters, device=dev))["p50"]
    print("SAME_BOX " + json.dumps({"workload": name, "config": config, "ours_ms": round(t_ours, 4),
                                     "reference_kernel_ms": round(t_ref, 4), "ratio": round(t_ref / t_ours, 2)}))


def _close(a, b, atol=2e-3, rtol=1e-2):
    a, b = a.float(), b.float()
    bad = (a - b).abs() > atol + rtol * b.abs()
    assert not bool(bad.any()), f"max |diff| {(a - b).abs().max().item():.3e}, {int(bad.sum())} of {bad.numel()} outside the band"


def _kv(B, H_kv, N, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn(B, H_kv, N, d, device="cuda", generator=g).half()
    v = torch.randn(B, H_kv, N, d, device="cuda", generator=g).half()
    return k, v, g


def test_paged_gqa_decode_fp16_against_v8_gqa_ss():
    from fa_kernels import gqa_attention
    from fa_kernels.paged import build_paged_kv
    ref = _reference_module("v8_gqa_ss")
    B, H_q, H_kv, N, d, page = 64, 32, 8, 4608, 128, 16
    k, v, g = _kv(B, H_kv, N, d, 2)
    q = torch.randn(B, H_q, 1, d, device="cuda", generator=g).half()
    kp, vp, bt, n_k = build_paged_kv(k, v, page, seed=2)
    scale = 1.0 / d ** 0.5
    ours = lambda: gqa_attention(q, kp, vp, bt, page, n_k)
    theirs = lambda: ref.forward(q, kp, vp, bt, page, int(n_k), scale, False, 0)
    _close(ours(), theirs())
    _time_both("paged_gqa_decode_fp16", ours, theirs, {"B": B, "h_q": H_q, "h_kv": H_kv, "n_k": N, "d": d, "page": page})


@pytest.mark.parametrize("fmt", ["e4m3", "nvfp4"])
def test_quantised_long_context_decode_against_v9_v10(fmt):
    import fa_kernels as F
    from fa_kernels import paged as P
    ref = _reference_module("v9_fp8" if fmt == "e4m3" else "v10_nvfp4")
    B, H_q, H_kv, N, d, page = 4, 32, 8, 131072, 128, 64
    k, v, g = _kv(B, H_kv, N, d, 4)
    q = torch.randn(B, H_q, 1, d, device="cuda", generator=g).half()
    scale = 1.0 / d ** 0.5
    if fmt == "e4m3":
        kp, vp, bt, n_k, sk, sv = P.build_paged_kv_fp8(k, v, page, seed=4)
        ours = lambda: F.fp8_attention(q, kp, vp, bt, page, n_k, sk, sv)
        theirs = lambda: ref.forward(q, kp, vp, bt, page, int(n_k), float(sk), float(sv), scale, False, 0)
    else:
        kp, km, vp, vm, bt, n_k, sk, sv = P.build_paged_kv_nvfp4(k, v, page, seed=4)
        ours = lambda: F.nvfp4_attention(q, kp, km, vp, vm, bt, page, n_k, sk, sv)
        theirs = lambda: ref.forward(q, kp, km, vp, vm, bt, page, int(n_k), float(sk), float(sv), scale, False, 0)
    del k, v
    _close(ours(), theirs())
    _time_both(f"long_decode_{fmt}", ours, theirs, {"B": B, "h_q": H_q, "h_kv": H_kv, "n_k": N, "d": d, "page": page,
                                                   "scales": "per tensor"})


def test_mla_decode_nvfp4_latent_against_v11_mla():
    import fa_kernels as F
    ref = _reference_module("v11_mla")
    B, H_q, N, dqk, dv, page = 16, 128, 16384, 576, 512, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    latent = torch.randn(B, 1, N, dqk, device="cuda", generator=g).half()
    q = torch.randn(B, H_q, 1, dqk, device="cuda", generator=g).half()
    lp, lm, bt, n_k, sl = F.build_paged_kv_mla(latent, page, seed=5)
    del latent
    scale = 1.0 / dqk ** 0.5
    ours = lambda: F.mla_attention(q, lp, lm, bt, page, n_k, dv, sl)
    theirs = lambda: ref.forward(q, lp, lm, bt, page, int(n_k), dv, float(sl), scale, False, 0)
    _close(ours(), theirs())
    _time_both("mla_decode_nvfp4_latent", ours, theirs, {"B": B, "h_q": H_q, "n_k": N, "dqk": dqk, "dv": dv, "page": page})


def test_causal_prefill_fp16_against_v5_wmma():
    from fa_kernels import attention
    ref = _reference_module("v5_wmma")
    B, H, N, d = 1, 32, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(1)
    q, k, v = (torch.randn(B, H, N, d, device="cuda", generator=g).half() for _ in range(3))
    scale = 1.0 / d ** 0.5
    ours = lambda: attention(q, k, v, causal=True)
    theirs = lambda: ref.forward(q, k, v, scale, True)
    _close(ours(), theirs())
    _time_both("causal_prefill_fp16", ours, theirs, {"B": B, "heads": H, "n": N, "d": d}, iters=3)
