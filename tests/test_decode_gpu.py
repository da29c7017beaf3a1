"""Parity of the paged GQA decode kernels (fp16 / bf16 / FP8 E4M3 / NVFP4 pools) with the oracle.

The shape matrix follows the reference's tests (tests/test_correctness.py:213-525 there): decode with
N_k in {4096, 8190}, G in {1,2,4,8}, d in {64,128}, idle-row G=3 and multi-tile G=16, the square
prefill through the paged path — plus what that suite never pins: per-sequence lengths, page sizes
16/64/48, LSE, fp16 output, per-token FP8 scales, bf16 pools.  Tolerance: max-abs 2e-3 + rel 1e-2
against the fp64 oracle fed the same stored values (every call goes through the C ABI).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import assert_close, dev, page, paged_varlen, perm_for, randn
from oracle import fa_oracle as O

pytestmark = pytest.mark.gpu


def _paged_inputs(B, H_kv, N_k, d, page_size, seed, dtype=torch.float16):
    _, k = randn((B, H_kv, N_k, d), seed * 10 + 1, dtype)
    _, v = randn((B, H_kv, N_k, d), seed * 10 + 2, dtype)
    n_logical = (N_k + page_size - 1) // page_size
    perm = perm_for(B * n_logical, seed)
    kp, vp, bt, _ = O.build_paged_kv(k, v, page_size, perm)
    return k, v, kp, vp, bt


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("N_k", [4096, 8190])
@pytest.mark.parametrize("G", [1, 2, 4, 8])
@pytest.mark.parametrize("causal", [False, True])
def test_gqa_decode(causal, G, N_k, d):
    from fa_kernels import gqa_attention
    B, H_kv, page_size = 1, 2, 128
    q_t, q = randn((B, G * H_kv, 1, d), 8)
    k, v, kp, vp, bt = _paged_inputs(B, H_kv, N_k, d, page_size, 8)
    q_offset = (N_k - 1) if causal else 0
    out = gqa_attention(q_t.cuda(), dev(kp, torch.float16), dev(vp, torch.float16), dev(bt), page_size, N_k,
                        causal=causal, q_offset=q_offset, backend="v8_gqa_ss")
    assert out.dtype == torch.float32 and tuple(out.shape) == (B, G * H_kv, 1, d)
    assert_close(out, O.gqa_attention_ref(q, k, v), what="gqa decode")


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("G", [3, 16])
def test_gqa_idle_rows_and_full_tile(G, d):
    from fa_kernels import gqa_attention
    B, H_kv, N_k, page_size = 1, 2, 8192, 256
    q_t, q = randn((B, G * H_kv, 1, d), 80)
    k, v, kp, vp, bt = _paged_inputs(B, H_kv, N_k, d, page_size, 80)
    out = gqa_attention(q_t.cuda(), dev(kp, torch.float16), dev(vp, torch.float16), dev(bt), page_size, N_k)
    assert_close(out, O.gqa_attention_ref(q, k, v), what="gqa idle/multi")


@pytest.mark.parametrize("causal", [False, True])
def test_gqa_square_prefill_through_paged_path(causal):
    from fa_kernels import gqa_attention
    B, H_kv, N, d, G, page_size = 2, 2, 512, 64, 4, 128
    q_t, q = randn((B, G * H_kv, N, d), 81)
    k, v, kp, vp, bt = _paged_inputs(B, H_kv, N, d, page_size, 81)
    out = gqa_attention(q_t.cuda(), dev(kp, torch.float16), dev(vp, torch.float16), dev(bt), page_size, N,
                        causal=causal, q_offset=0)
    assert_close(out, O.gqa_attention_ref(q, k, v, causal=causal), what="gqa square")


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("N_k", [4096, 8190])
@pytest.mark.parametrize("page_size", [128, 256])
@pytest.mark.parametrize("causal", [False, True])
def test_paged_mha_decode(causal, page_size, N_k, d):
    from fa_kernels import paged_attention
    B, H = 1, 8
    q_t, q = randn((B, H, 1, d), 6)
    k, v, kp, vp, bt = _paged_inputs(B, H, N_k, d, page_size, 6)
    out = paged_attention(q_t.cuda(), dev(kp, torch.float16), dev(vp, torch.float16), dev(bt), page_size, N_k,
                          causal=causal, q_offset=(N_k - 1) if causal else 0)
    assert_close(out, O.attention_ref(q, k, v), what="paged decode")


def test_fp32_inputs_are_accepted_like_the_reference():
    """The reference casts fp32 q / pools to half on entry (gqa_ss_attention.cu:293-295); the result
    then sits in its 2e-2 band against the fp32 oracle on the unrounded inputs."""
    from fa_kernels import gqa_attention
    B, H_kv, G, N_k, d, page_size = 1, 2, 4, 4096, 128, 128
    q_t, q = randn((B, G * H_kv, 1, d), 8, torch.float32)
    k, v, kp, vp, bt = _paged_inputs(B, H_kv, N_k, d, page_size, 8, torch.float32)
    out = gqa_attention(q_t.cuda(), dev(kp, torch.float32), dev(vp, torch.float32), dev(bt), page_size, N_k)
    assert_close(out, O.gqa_attention_ref(q, k, v), atol=2e-2, rtol=2e-2, what="fp32 in")


@pytest.mark.parametrize("page_size", [16, 64, 48])
@pytest.mark.parametrize("d", [64, 128])
def test_varlen_pages_lse_and_fp16_out(page_size, d):
    from fa_kernels import gqa_attention
    H_kv, G = 2, 4
    lens = [1, 15, 16, 17, 0, 1000, 4097, 63, 64, 65]
    B = len(lens)
    q_t, q = randn((B, G * H_kv, 1, d), 31)
    ks = [randn((H_kv, n, d), 100 + i)[1] for i, n in enumerate(lens)]
    vs = [randn((H_kv, n, d), 200 + i)[1] for i, n in enumerate(lens)]
    kp, bt, perm = paged_varlen(ks, page_size, 31)
    vp, bt2, _ = paged_varlen(vs, page_size, 31)
    assert (bt == bt2).all()
    out, lse = gqa_attention(q_t.cuda(), dev(kp, torch.float16), dev(vp, torch.float16), dev(bt), page_size, lens,
                             out_dtype=torch.float16, return_lse=True)
    assert out.dtype == torch.float16
    ref, ref_lse = O.paged_gqa_attention_ref(q, kp, vp, bt, page_size, lens, return_lse=True)
    assert_close(out, ref, what="varlen out")
    fin = np.isfinite(ref_lse)
    got = lse.cpu().numpy()
    assert (np.isneginf(got) == ~fin).all()
    np.testing.assert_allclose(got[fin], ref_lse[fin], atol=2e-3, rtol=1e-3)
    assert (out[4] == 0).all()        # the empty sequence returns zeros


def test_host_buffer_step_matches_device_api_and_oracle():
    """fa_paged_decode_host through HostDecodeStep: q, block table and lengths start in pinned host memory,
    the output ends there; three steps in a row with different lengths (long enough to be split, ragged,
    empty) reuse the staging buffers and must equal the device-tensor API bit for bit."""
    from fa_kernels import HostDecodeStep, gqa_attention
    H_kv, G, d, page_size = 2, 4, 128, 16
    all_lens = [[1000, 4097, 63, 0], [16, 17, 9000, 5], [4096, 4096, 4096, 4096]]
    B = 4
    ks = [randn((H_kv, 9000, d), 300 + i)[1] for i in range(B)]
    vs = [randn((H_kv, 9000, d), 400 + i)[1] for i in range(B)]
    kp, bt, _ = paged_varlen(ks, page_size, 33)
    vp, _, _ = paged_varlen(vs, page_size, 33)
    kp_d, vp_d = dev(kp, torch.float16), dev(vp, torch.float16)
    bt_t = torch.from_numpy(np.ascontiguousarray(bt)).to(torch.int32)
    step = HostDecodeStep(kp_d, vp_d, page_size, B, G * H_kv, 1, d, bt_t.shape[1], out_dtype=torch.float16)
    bt_host = bt_t.pin_memory()
    out_host = torch.empty((B, G * H_kv, 1, d), dtype=torch.float16).pin_memory()
    for it, lens in enumerate(all_lens):
        q_t, q = randn((B, G * H_kv, 1, d), 50 + it)
        q_host = q_t.to(torch.float16).pin_memory()
        step(q_host, bt_host, torch.tensor(lens, dtype=torch.int32).pin_memory(), out_host)
        torch.cuda.current_stream().synchronize()
        same = gqa_attention(q_t.cuda(), kp_d, vp_d, bt_t.cuda(), page_size, lens, out_dtype=torch.float16)
        assert torch.equal(out_host, same.cpu())
        ref = O.paged_gqa_attention_ref(q, kp, vp, bt, page_size, lens)
        assert_close(out_host, ref, what=f"host step {it}")


def test_split_count_does_not_change_the_result():
    from fa_kernels import gqa_attention
    B, H_kv, G, N_k, d, page_size = 2, 2, 4, 8190, 128, 16
    q_t, q = randn((B, G * H_kv, 1, d), 41)
    k, v, kp, vp, bt = _paged_inputs(B, H_kv, N_k, d, page_size, 41)
    args = (q_t.cuda(), dev(kp, torch.float16), dev(vp, torch.float16), dev(bt), page_size, N_k)
    ref = O.gqa_attention_ref(q, k, v)
    outs = [gqa_attention(*args, chunk_hint=c) for c in (64, 256, 1024, 100000)]
    for o in outs:
        assert_close(o, ref, what="split invariance")
    # repeated calls reuse the self-resetting arrival counters
    assert torch.equal(gqa_attention(*args, chunk_hint=256), outs[1])


def test_bf16_pools():
    from fa_kernels import gqa_attention
    B, H_kv, G, N_k, d, page_size = 2, 2, 4, 3000, 128, 64
    q_t, q = randn((B, G * H_kv, 1, d), 51, torch.bfloat16)
    k, v, kp, vp, bt = _paged_inputs(B, H_kv, N_k, d, page_size, 51, torch.bfloat16)
    out = gqa_attention(q_t.cuda(), dev(kp, torch.bfloat16), dev(vp, torch.bfloat16), dev(bt), page_size, N_k,
                        out_dtype=torch.bfloat16)
    assert_close(out, O.gqa_attention_ref(q, k, v), what="bf16")


# ---------------------------------------------------------------------------------------------- FP8
def _fp8_case(B, H_kv, G, N_k, d, page_size, seed, per_token):
    q_t, q = randn((B, G * H_kv, 1 if isinstance(N_k, int) else 1, d), seed)
    _, k = randn((B, H_kv, N_k, d), seed * 10 + 1, torch.float32)
    _, v = randn((B, H_kv, N_k, d), seed * 10 + 2, torch.float32)
    return q_t, q, k.astype(np.float32), v.astype(np.float32)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("N_k", [4096, 8190])
@pytest.mark.parametrize("G", [1, 2, 4, 8])
@pytest.mark.parametrize("causal", [False, True])
def test_fp8_decode_per_tensor(causal, G, N_k, d):
    from fa_kernels import fp8_attention
    B, H_kv, page_size = 1, 2, 128
    q_t, q, k, v = _fp8_case(B, H_kv, G, N_k, d, page_size, 9, False)
    kb, sk = O.quantize_fp8_e4m3(k)
    vb, sv = O.quantize_fp8_e4m3(v)
    perm = perm_for(B * ((N_k + page_size - 1) // page_size), 9)
    kp, vp, bt, _ = O.build_paged_kv(kb, vb, page_size, perm)
    out = fp8_attention(q_t.cuda(), dev(kp), dev(vp), dev(bt), page_size, N_k, sk, sv,
                        causal=causal, q_offset=(N_k - 1) if causal else 0)
    ref = O.gqa_attention_ref(q, O.dequantize_fp8_e4m3(kb, sk), O.dequantize_fp8_e4m3(vb, sv))
    assert_close(out, ref, what="fp8 per-tensor")
    rmse = float(np.sqrt(np.mean((out.cpu().numpy() - O.gqa_attention_ref(q, k, v)) ** 2)))
    assert rmse < 0.5


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("G", [3, 4, 16])
def test_fp8_decode_per_token_scales(G, d):
    """One fp32 scale per token per head, keys with x10 outlier channels (the long-context layout)."""
    from fa_kernels import fp8_attention
    B, H_kv, N_k, page_size = 2, 2, 5000, 64
    q_t, q, k, v = _fp8_case(B, H_kv, G, N_k, d, page_size, 90, True)
    k[..., 5] *= 10.0
    v[..., 17] *= 10.0
    kb, ks = O.quantize_fp8_e4m3_per_token(k)
    vb, vs = O.quantize_fp8_e4m3_per_token(v)
    perm = perm_for(B * ((N_k + page_size - 1) // page_size), 90)
    kp, vp, bt, _ = O.build_paged_kv(kb, vb, page_size, perm)
    ksp, vsp, _, _ = O.build_paged_kv(ks[..., None], vs[..., None], page_size, perm)
    out = fp8_attention(q_t.cuda(), dev(kp), dev(vp), dev(bt), page_size, N_k, dev(ksp[..., 0]), dev(vsp[..., 0]))
    ref = O.gqa_attention_ref(q, O.e4m3_decode(kb) * ks[..., None], O.e4m3_decode(vb) * vs[..., None])
    assert_close(out, ref, what="fp8 per-token")


@pytest.mark.parametrize("per_token", [False, True])
@pytest.mark.parametrize("G", [1, 4, 5, 8])
def test_fp8_tcgen05_and_mma_sync_kernels_agree(G, per_token):
    """Pages of 64 tokens and one query position put E4M3 pools on the tcgen05 kernel (keys as the M dimension,
    csrc/decode_tc.cu); variant=9 keeps the mma.sync kernel.  Both against the oracle, on ragged per-sequence
    lengths that cover less than one tile (100 keys), a tile boundary (128), an odd tile count, a long sequence
    that is split into key ranges, and a causal limit inside the sequence."""
    from fa_kernels import fp8_attention
    H_kv, d, page_size = 2, 128, 64
    lens = [100, 128, 129, 1000, 9001]
    B, N_max = len(lens), max(lens)
    q_t, q, k, v = _fp8_case(B, H_kv, G, N_max, d, page_size, 77 + G, per_token)
    k[..., 9] *= 10.0
    if per_token:
        kb, ks = O.quantize_fp8_e4m3_per_token(k)
        vb, vs = O.quantize_fp8_e4m3_per_token(v)
        k_hat, v_hat = O.e4m3_decode(kb) * ks[..., None], O.e4m3_decode(vb) * vs[..., None]
    else:
        kb, sk = O.quantize_fp8_e4m3(k)
        vb, sv = O.quantize_fp8_e4m3(v)
        k_hat, v_hat = O.dequantize_fp8_e4m3(kb, sk), O.dequantize_fp8_e4m3(vb, sv)
    perm = perm_for(B * ((N_max + page_size - 1) // page_size), 77)
    kp, vp, bt, _ = O.build_paged_kv(kb, vb, page_size, perm)
    if per_token:
        ksp, vsp, _, _ = O.build_paged_kv(ks[..., None], vs[..., None], page_size, perm)
        scales = (dev(ksp[..., 0]), dev(vsp[..., 0]))
    else:
        scales = (sk, sv)
    for causal, q_off in ((False, 0), (True, 70)):
        outs = {}
        for variant in (0, 9):
            out, lse = fp8_attention(q_t.cuda(), dev(kp), dev(vp), dev(bt), page_size, lens, *scales, causal=causal,
                                     q_offset=q_off, return_lse=True, variant=variant)
            outs[variant] = out
            for b, n in enumerate(lens):
                n_eff = min(n, q_off + 1) if causal else n
                ref, ref_lse = O.gqa_attention_ref(q[b:b + 1], k_hat[b:b + 1, :, :n_eff], v_hat[b:b + 1, :, :n_eff], return_lse=True)
                assert_close(out[b:b + 1], ref, what=f"fp8 variant {variant} seq {b} causal {causal}")
                np.testing.assert_allclose(lse[b:b + 1].cpu().numpy(), ref_lse, atol=3e-3, rtol=1e-3)
        assert_close(outs[0], outs[9].cpu().numpy(), what="tcgen05 vs mma.sync")


def test_fp8_tcgen05_rising_scores_and_zero_tokens():
    """Scores that keep rising along the sequence (the running maximum is raised in many tiles, so the output
    accumulator is rescaled again and again), queries eight times the usual magnitude, and tokens whose K and V
    rows are all zero (their per-token scale is the quantiser's floor): tcgen05 and mma.sync kernels against
    the oracle."""
    from fa_kernels import fp8_attention
    B, H_kv, G, N_k, d, page_size = 2, 2, 4, 6000, 128, 64
    q_t, q, k, v = _fp8_case(B, H_kv, G, N_k, d, page_size, 123, True)
    q_t, q = q_t * 8.0, q * 8.0
    ramp = np.linspace(0.0, 1.0, N_k, dtype=np.float32)[None, None, :, None]
    k = k * 0.05 + ramp * np.sign(q[:, ::G, :1, :]) * 0.5            # the dot product with q grows with the position
    k[:, :, 100:140] = 0.0
    v[:, :, 100:140] = 0.0
    v[:, :, 4000:4003] = 0.0
    kb, ks = O.quantize_fp8_e4m3_per_token(k)
    vb, vs = O.quantize_fp8_e4m3_per_token(v)
    perm = perm_for(B * ((N_k + page_size - 1) // page_size), 123)
    kp, vp, bt, _ = O.build_paged_kv(kb, vb, page_size, perm)
    ksp, vsp, _, _ = O.build_paged_kv(ks[..., None], vs[..., None], page_size, perm)
    ref, ref_lse = O.gqa_attention_ref(q, O.e4m3_decode(kb) * ks[..., None], O.e4m3_decode(vb) * vs[..., None], return_lse=True)
    for variant in (0, 9):
        out, lse = fp8_attention(q_t.cuda(), dev(kp), dev(vp), dev(bt), page_size, N_k, dev(ksp[..., 0]), dev(vsp[..., 0]),
                                 return_lse=True, variant=variant)
        assert_close(out, ref, what=f"fp8 rising scores, variant {variant}")
        np.testing.assert_allclose(lse.cpu().numpy(), ref_lse, atol=3e-3, rtol=1e-3)


# -------------------------------------------------------------------------------------------- NVFP4
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("N_k", [4096, 8190])
@pytest.mark.parametrize("G", [1, 2, 4, 8])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("seed", [9, 17])
def test_nvfp4_decode(seed, causal, G, N_k, d):
    from fa_kernels import nvfp4_attention
    B, H_kv, page_size = 1, 2, 128
    q_t, q, k, v = _fp8_case(B, H_kv, G, N_k, d, page_size, seed, False)
    kpk, kmi, sk = O.quantize_nvfp4(k)
    vpk, vmi, sv = O.quantize_nvfp4(v)
    perm = perm_for(B * ((N_k + page_size - 1) // page_size), seed)
    kp, vp, bt, _ = O.build_paged_kv(kpk, vpk, page_size, perm)
    km, vm, _, _ = O.build_paged_kv(kmi, vmi, page_size, perm)
    out = nvfp4_attention(q_t.cuda(), dev(kp), dev(km), dev(vp), dev(vm), dev(bt), page_size, N_k, sk, sv,
                          causal=causal, q_offset=(N_k - 1) if causal else 0)
    ref = O.gqa_attention_ref(q, O.dequantize_nvfp4(kpk, kmi, sk), O.dequantize_nvfp4(vpk, vmi, sv))
    assert_close(out, ref, what="nvfp4")
    rmse = float(np.sqrt(np.mean((out.cpu().numpy() - O.gqa_attention_ref(q, k, v)) ** 2)))
    assert rmse < 0.8


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("G", [3, 16])
def test_nvfp4_idle_rows_full_tile_small_pages(G, d):
    from fa_kernels import nvfp4_attention
    B, H_kv, N_k, page_size = 2, 2, 2500, 16
    q_t, q, k, v = _fp8_case(B, H_kv, G, N_k, d, page_size, 100, False)
    k[..., 3] *= 10.0
    kpk, kmi, sk = O.quantize_nvfp4(k)
    vpk, vmi, sv = O.quantize_nvfp4(v)
    perm = perm_for(B * ((N_k + page_size - 1) // page_size), 100)
    kp, vp, bt, _ = O.build_paged_kv(kpk, vpk, page_size, perm)
    km, vm, _, _ = O.build_paged_kv(kmi, vmi, page_size, perm)
    out = nvfp4_attention(q_t.cuda(), dev(kp), dev(km), dev(vp), dev(vm), dev(bt), page_size, N_k, sk, sv)
    ref = O.gqa_attention_ref(q, O.dequantize_nvfp4(kpk, kmi, sk), O.dequantize_nvfp4(vpk, vmi, sv))
    assert_close(out, ref, what="nvfp4 G/pages")


@pytest.mark.parametrize("fmt", ["e4m3", "nvfp4"])
@pytest.mark.parametrize("causal", [False, True])
def test_quantised_square_prefill(causal, fmt):
    from fa_kernels import fp8_attention, nvfp4_attention
    B, H_kv, N, d, G, page_size = 2, 2, 512, 64, 4, 128
    q_t, q = randn((B, G * H_kv, N, d), 91)
    _, k = randn((B, H_kv, N, d), 911, torch.float32)
    _, v = randn((B, H_kv, N, d), 912, torch.float32)
    k, v = k.astype(np.float32), v.astype(np.float32)
    perm = perm_for(B * (N // page_size), 91)
    if fmt == "e4m3":
        kb, sk = O.quantize_fp8_e4m3(k)
        vb, sv = O.quantize_fp8_e4m3(v)
        kp, vp, bt, _ = O.build_paged_kv(kb, vb, page_size, perm)
        out = fp8_attention(q_t.cuda(), dev(kp), dev(vp), dev(bt), page_size, N, sk, sv, causal=causal)
        ref = O.gqa_attention_ref(q, O.dequantize_fp8_e4m3(kb, sk), O.dequantize_fp8_e4m3(vb, sv), causal=causal)
    else:
        kpk, kmi, sk = O.quantize_nvfp4(k)
        vpk, vmi, sv = O.quantize_nvfp4(v)
        kp, vp, bt, _ = O.build_paged_kv(kpk, vpk, page_size, perm)
        km, vm, _, _ = O.build_paged_kv(kmi, vmi, page_size, perm)
        out = nvfp4_attention(q_t.cuda(), dev(kp), dev(km), dev(vp), dev(vm), dev(bt), page_size, N, sk, sv,
                              causal=causal)
        ref = O.gqa_attention_ref(q, O.dequantize_nvfp4(kpk, kmi, sk), O.dequantize_nvfp4(vpk, vmi, sv), causal=causal)
    assert_close(out, ref, what=f"{fmt} square")


# ------------------------------------------------------------------------------------------- merge
def test_merge_partials_matches_oracle():
    from fa_kernels._decode import merge_partials
    g = torch.Generator().manual_seed(5)
    o = torch.randn(5, 3, 7, 128, generator=g)
    l = torch.randn(5, 3, 7, generator=g) * 3
    l[2] = float("-inf")                 # an empty key range
    l[:, 1, 3] = float("-inf")           # a row with no keys anywhere
    out, lse = merge_partials(o.cuda(), l.cuda(), return_lse=True)
    ref, ref_lse = O.merge_partials_ref(o.numpy(), l.numpy())
    assert_close(out, ref, atol=1e-5, rtol=1e-5, what="merge")
    fin = np.isfinite(ref_lse)
    np.testing.assert_allclose(lse.cpu().numpy()[fin], ref_lse[fin], atol=1e-5)
    assert np.isneginf(lse.cpu().numpy()[~fin]).all()


# ------------------------------------------------------------------------------------------ errors
def test_error_behaviour_matches_reference_contract():
    from fa_kernels import gqa_attention
    q = torch.zeros(1, 4, 1, 128, device="cuda", dtype=torch.float16)
    pool = torch.zeros(4, 16, 2, 128, device="cuda", dtype=torch.float16)
    bt = torch.zeros(1, 4, device="cuda", dtype=torch.int32)
    with pytest.raises(KeyError):
        gqa_attention(q, pool, pool, bt, 16, 64, backend="v99_nope")
    with pytest.raises(RuntimeError, match="int32"):
        gqa_attention(q, pool, pool, bt.long(), 16, 64)
    with pytest.raises(RuntimeError, match="cover"):
        gqa_attention(q, pool, pool, bt, 16, 65)
    with pytest.raises(RuntimeError, match="multiple of H_kv"):
        gqa_attention(q[:, :3], pool, pool, bt, 16, 64)
    with pytest.raises(RuntimeError, match="head_dim"):
        gqa_attention(q[..., :32].contiguous(), pool[..., :32].contiguous(), pool[..., :32].contiguous(), bt, 16, 64)
    with pytest.raises(RuntimeError, match="page_size"):
        gqa_attention(q, pool, pool, bt, 32, 64)


# ------------------------------------------------------------- KV-range shards, emulated on one GPU
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("world", [2, 8])
def test_kv_range_shards_merge_to_the_full_result(world, causal):
    """What each rank of a KV-range-sharded decode computes (local pool slice, q_offset shifted by the
    range start, output and LSE written into one flat send buffer) followed by the strided merge of
    the gathered buffer — all ranks played in turn by one GPU, the all-gather replaced by a copy."""
    from fa_kernels import gqa_attention
    from fa_kernels._decode import merge_partials
    from fa_kernels.distributed import kv_range_shards
    B, H_kv, G, N_q, N_k, d, page = 2, 2, 4, 2, 3000, 128, 64
    q_t, q = randn((B, G * H_kv, N_q, d), 61)
    _, k = randn((B, H_kv, N_k, d), 611)
    _, v = randn((B, H_kv, N_k, d), 612)
    q_offset = N_k - N_q
    rows, D = B * G * H_kv * N_q, d
    recv = torch.empty(world, rows * (D + 1), dtype=torch.float32, device="cuda")
    for r, (kb, ke) in enumerate(kv_range_shards(N_k, page, world)):
        n = ke - kb
        n_logical = max((n + page - 1) // page, 1)
        perm = perm_for(B * n_logical, 61 + r)
        kp, vp, bt, _ = O.build_paged_kv(np.ascontiguousarray(k[:, :, kb:ke]), np.ascontiguousarray(v[:, :, kb:ke]), page, perm) \
            if n > 0 else (np.zeros((B, page, H_kv, d)), np.zeros((B, page, H_kv, d)), np.zeros((B, 1), np.int32), 0)
        send = recv[r]
        gqa_attention(q_t.cuda(), dev(kp, torch.float16), dev(vp, torch.float16), dev(bt), page, n, causal=causal,
                      q_offset=q_offset - kb, out_dtype=torch.float32,
                      out=send[: rows * D].view(B, G * H_kv, N_q, D), lse_out=send[rows * D:].view(B, G * H_kv, N_q))
    out, lse = merge_partials(recv[:, : rows * D].unflatten(1, (B, G * H_kv, N_q, D)),
                              recv[:, rows * D:].unflatten(1, (B, G * H_kv, N_q)), return_lse=True)
    ref, ref_lse = O.gqa_attention_ref(q, k, v, causal=causal, q_offset=q_offset, return_lse=True)
    assert_close(out, ref, what="kv-range merge")
    np.testing.assert_allclose(lse.cpu().numpy(), ref_lse, atol=2e-3, rtol=1e-3)
