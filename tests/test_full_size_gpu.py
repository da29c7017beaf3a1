"""The benchmark configurations at their full sizes against the oracle.

Split planning, block-table staging and 32-bit offsets behave differently at 300 000-token batches, at
1 048 576-key contexts and at 128 x 32 768-key latents than at the few-thousand-key shapes of the other
tests, so each configuration is run once as the benchmark runs it and a sample of its output is compared
with the fp64 oracle on the very bytes the kernel read (gathered from the pools with plain torch indexing,
not with the library's own gather).  Inputs are generated on the GPU with the benchmark's seeds.
"""

from __future__ import annotations

import importlib.util
import os

import numpy as np
import pytest
import torch

from conftest import PKG_DIR
from helpers import assert_close
from oracle import fa_oracle as O

pytestmark = pytest.mark.gpu


def _rows_of(pool, bt_row, page, n):
    """Logical tokens [0, n) of one sequence: [n, H, dx] (torch indexing; independent of fa_paged_gather)."""
    pages = pool[bt_row[: (n + page - 1) // page].long()]
    return pages.reshape(-1, *pool.shape[2:])[:n]


def test_paged_gqa_decode_batch_64_every_sequence():
    """fp16, batch 64, 32 / 8 heads, d 128, contexts uniform in [1024, 8192], 16-token pages: all 64
    sequences, output and LSE."""
    from fa_bench import workloads
    from fa_kernels import check_status, gqa_attention
    w = workloads.paged_gqa_decode(torch.device("cuda"), seed=2)
    assert len(w["seq_lens"]) == 64 and 1024 <= min(w["seq_lens"]) and max(w["seq_lens"]) <= 8192
    out, lse = gqa_attention(w["q"], w["k_pool"], w["v_pool"], w["block_table"], 16, w["seq_lens"], out_dtype=torch.float16,
                             return_lse=True)
    check_status()
    q = w["q"].float().cpu().numpy().astype(np.float64)
    for b, n in enumerate(w["seq_lens"]):
        k = _rows_of(w["k_pool"], w["block_table"][b], 16, n).float().cpu().numpy().transpose(1, 0, 2)
        v = _rows_of(w["v_pool"], w["block_table"][b], 16, n).float().cpu().numpy().transpose(1, 0, 2)
        ref, ref_lse = O.gqa_attention_ref(q[b:b + 1], k[None], v[None], return_lse=True)
        assert_close(out[b:b + 1], ref, what=f"batch-64 decode, sequence {b} ({n} keys)")
        np.testing.assert_allclose(lse[b:b + 1].cpu().numpy(), ref_lse, atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("fmt", ["e4m3", "nvfp4"])
def test_long_context_decode_one_million_keys(fmt):
    """B=4, 32 / 8 heads, d 128, context 1 048 576, page 64, 1 % of the channels x10: one (sequence, KV
    head) slice over all its keys, output and LSE, against the oracle's dequantisation of the stored bytes.
    Every other slice must be finite and inside the convex hull of its values."""
    from fa_bench import workloads
    from fa_kernels import check_status, fp8_attention, nvfp4_attention
    w = workloads.quantised_long_context_decode(torch.device("cuda"), fmt=fmt)
    n, page = w["n_k"], 64
    assert n == 1048576 and w["q"].shape == (4, 32, 1, 128)
    if fmt == "e4m3":
        out, lse = fp8_attention(w["q"], w["k_pool"], w["v_pool"], w["block_table"], page, n, w["k_scale"], w["v_scale"],
                                 out_dtype=torch.float16, return_lse=True)
    else:
        out, lse = nvfp4_attention(w["q"], w["k_pool"], w["k_micro"], w["v_pool"], w["v_micro"], w["block_table"], page, n,
                                   w["k_scale"], w["v_scale"], out_dtype=torch.float16, return_lse=True)
    check_status()
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    b, h = (2, 5) if fmt == "e4m3" else (3, 1)
    bt = w["block_table"][b]

    def slice_of(pool):            # [n, dx] of head h
        return _rows_of(pool[:, :, h:h + 1], bt, page, n)[:, 0].cpu().numpy()
    if fmt == "e4m3":
        ks = _rows_of(w["k_scale"][:, :, h:h + 1, None], bt, page, n)[:, 0].cpu().numpy()
        vs = _rows_of(w["v_scale"][:, :, h:h + 1, None], bt, page, n)[:, 0].cpu().numpy()
        k = O.e4m3_decode(slice_of(w["k_pool"])).astype(np.float64) * ks
        v = O.e4m3_decode(slice_of(w["v_pool"])).astype(np.float64) * vs
    else:
        k = O.dequantize_nvfp4(slice_of(w["k_pool"]), slice_of(w["k_micro"]), w["k_scale"]).astype(np.float64)
        v = O.dequantize_nvfp4(slice_of(w["v_pool"]), slice_of(w["v_micro"]), w["v_scale"]).astype(np.float64)
    # the four query heads of the group as four query rows over the one KV head (no mask: same arithmetic)
    q = w["q"][b, 4 * h:4 * h + 4, 0].float().cpu().numpy().astype(np.float64)[None, None]
    ref, ref_lse = O.attention_ref(q, k[None, None], v[None, None], return_lse=True)
    assert_close(out[b, 4 * h:4 * h + 4, 0], ref[0, 0], what=f"1 Mi-key {fmt} decode, sequence {b} head {h}")
    np.testing.assert_allclose(lse[b, 4 * h:4 * h + 4, 0].cpu().numpy(), ref_lse[0, 0], atol=2e-3, rtol=1e-3)
    assert float(out[b, 4 * h:4 * h + 4].float().abs().max()) <= float(np.abs(v).max()) + 1e-3


@pytest.mark.parametrize("latent", ["bf16", "e4m3"])
def test_mla_decode_batch_128_sampled_sequences(latent):
    """128 heads, latent 576 / 512, batch 128, contexts uniform in [4096, 32768], page 64: eight sequences
    including the longest and the shortest, output and LSE; all others finite."""
    from fa_bench import workloads
    from fa_kernels import check_status, mla_attention
    w = workloads.mla_decode(torch.device("cuda"), latent=latent)
    lens = w["seq_lens"]
    assert len(lens) == 128 and min(lens) >= 4096 and max(lens) <= 32768
    out, lse = mla_attention(w["q"], w["l_pool"], None, w["block_table"], 64, lens, 512, w["scale_l"], return_lse=True,
                             out_dtype=torch.float32)
    check_status()
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    order = sorted(range(128), key=lambda i: lens[i])
    sample = sorted({order[0], order[-1], order[1], order[-2], order[64], 0, 77, 127})
    for b in sample:
        n = lens[b]
        rows = _rows_of(w["l_pool"], w["block_table"][b], 64, n)[:, 0]
        if latent == "bf16":
            lat = rows.float().cpu().numpy().astype(np.float64)
        else:
            sc = _rows_of(w["scale_l"][..., None], w["block_table"][b], 64, n)[:, 0].cpu().numpy()
            lat = O.e4m3_decode(rows.cpu().numpy()).astype(np.float64) * sc
        # MQA over one latent (reference.py:100-111): the 128 heads as 128 query rows of one head, which
        # spares the oracle a 128-fold copy of the latent
        q = w["q"][b, :, 0].float().cpu().numpy().astype(np.float64)[None, None]
        ref, ref_lse = O.attention_ref(q, lat[None, None], lat[None, None, :, :512], scale=1.0 / 576 ** 0.5, return_lse=True)
        assert_close(out[b, :, 0], ref[0, 0], what=f"MLA {latent}, sequence {b} ({n} keys)")
        np.testing.assert_allclose(lse[b, :, 0].cpu().numpy(), ref_lse[0, 0], atol=3e-3, rtol=1e-3)


def test_reference_command_line_sweep_runs_one_small_shape(tmp_path):
    """fa_bench/sweep.py with the reference harness's flags, one small decode shape and one prefill shape:
    rows carry the columns of the reference's tables."""
    spec = importlib.util.spec_from_file_location("fa_sweep_cli", os.path.join(PKG_DIR, "fa_bench", "sweep.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = tmp_path / "rows.json"
    rows = mod.run(mod.build_parser().parse_args(
        f"--backend v8_gqa_ss --decode --seq 2048 --heads 8 --gqa-group 4 --dim 128 --page-size 16 --batch 2 --iters 3 --json {out}".split()))
    assert len(rows) == 1 and rows[0]["kv_gbs"] > 0 and rows[0]["us_per_token"] > 0 and out.exists()
    rows = mod.run(mod.build_parser().parse_args("--backend v5_wmma --seq 512 --heads 4 --dim 64 --causal --iters 3".split()))
    assert len(rows) == 1 and rows[0]["tflops"] > 0
