"""Parity of the MLA latent decode kernel with the oracle.

Matrix of the reference's MLA tests (tests/test_correctness.py:540-752 there): h_q in {16,32,64,128}
on the small latent (DQK 96 = 64 + 32), idle rows h_q in {3, 20}, the real (576, 512) latent at
h_q = 128, the square prefill, the absorption identity, and the engine-selecting entry point — all on
the NVFP4 latent of build_paged_kv_mla — plus bf16 and FP8 E4M3 (per-token scales) latents with
per-sequence lengths.  Oracle = MQA over the dequantised stored bytes in fp64; tolerance 2e-3 + 1e-2."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import assert_close, dev, paged_varlen, perm_for, randn
from oracle import fa_oracle as O

pytestmark = pytest.mark.gpu


def _nvfp4_latent(B, N_k, DQK, page_size, seed, scale=1.0):
    _, lat = randn((B, 1, N_k, DQK), seed * 10 + 1, torch.float32, scale)
    lat = lat.astype(np.float32)
    pk, mi, sl = O.quantize_nvfp4(lat)
    perm = perm_for(B * ((N_k + page_size - 1) // page_size), seed)
    lp, lm, bt, _ = O.build_paged_kv(pk, mi, page_size, perm)
    return lat, O.dequantize_nvfp4(pk, mi, sl), lp, lm, bt, sl


@pytest.mark.parametrize("N_k", [4096, 8190])
@pytest.mark.parametrize("h_q", [16, 32, 64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("seed", [9, 17])
def test_mla_decode_nvfp4_latent(seed, causal, h_q, N_k):
    from fa_kernels import mla_attention
    L, R, page_size = 64, 32, 128
    q_t, q = randn((1, h_q, 1, L + R), seed)
    _, lat_hat, lp, lm, bt, sl = _nvfp4_latent(1, N_k, L + R, page_size, seed)
    out = mla_attention(q_t.cuda(), dev(lp), dev(lm), dev(bt), page_size, N_k, L, sl, causal=causal,
                        q_offset=(N_k - 1) if causal else 0)
    assert out.dtype == torch.float32 and tuple(out.shape) == (1, h_q, 1, L)
    assert_close(out, O.mla_attention_ref(q, lat_hat, L), what="mla nvfp4")


@pytest.mark.parametrize("h_q", [3, 20])
def test_mla_idle_rows(h_q):
    from fa_kernels import mla_attention
    L, R, page_size, N_k = 64, 32, 256, 8192
    q_t, q = randn((1, h_q, 1, L + R), 100)
    _, lat_hat, lp, lm, bt, sl = _nvfp4_latent(1, N_k, L + R, page_size, 100)
    out = mla_attention(q_t.cuda(), dev(lp), dev(lm), dev(bt), page_size, N_k, L, sl)
    assert_close(out, O.mla_attention_ref(q, lat_hat, L), what="mla idle")


@pytest.mark.parametrize("N_k", [4096, 8190])
@pytest.mark.parametrize("engine", [None, "fp8", "nvfp4"])
def test_mla_real_shape(N_k, engine):
    from fa_kernels import mla_attention, mla_tc_attention
    h_q, L, R, page_size = 128, 512, 64, 128
    q_t, q = randn((1, h_q, 1, L + R), 7)
    _, lat_hat, lp, lm, bt, sl = _nvfp4_latent(1, N_k, L + R, page_size, 7)
    args = (q_t.cuda(), dev(lp), dev(lm), dev(bt), page_size, N_k, L, sl)
    out = mla_attention(*args) if engine is None else mla_tc_attention(*args, engine=engine)
    assert_close(out, O.mla_attention_ref(q, lat_hat, L), what="mla real shape")


@pytest.mark.parametrize("causal", [False, True])
def test_mla_square_prefill(causal):
    from fa_kernels import mla_attention
    h_q, N, L, R, page_size = 8, 512, 64, 32, 128
    q_t, q = randn((1, h_q, N, L + R), 101)
    _, lat_hat, lp, lm, bt, sl = _nvfp4_latent(1, N, L + R, page_size, 101)
    out = mla_attention(q_t.cuda(), dev(lp), dev(lm), dev(bt), page_size, N, L, sl, causal=causal, q_offset=0)
    assert_close(out, O.mla_attention_ref(q, lat_hat, L, causal=causal), what="mla square")


@pytest.mark.parametrize("h_q", [16, 64])
def test_mla_absorption_identity(h_q):
    """reference tests/test_correctness.py:624-658: the absorbed kernel re-projected through W_UV equals
    attention over the explicitly materialised per-head K / V."""
    from fa_kernels import mla_attention
    N_k, Dn, R, L, Dv, page_size = 4096, 48, 32, 64, 40, 128
    g = np.random.default_rng(5)
    q_nope = g.standard_normal((1, h_q, 1, Dn))
    q_rope = g.standard_normal((1, h_q, 1, R))
    W_UK = g.standard_normal((h_q, Dn, L)) / L ** 0.5
    W_UV = g.standard_normal((h_q, Dv, L)) / L ** 0.5
    q_abs = np.concatenate([np.einsum("bhnd,hdl->bhnl", q_nope, W_UK), q_rope], -1)
    q_t = torch.from_numpy(q_abs).half()
    q_abs = q_t.float().numpy().astype(np.float64)
    _, lat_hat, lp, lm, bt, sl = _nvfp4_latent(1, N_k, L + R, page_size, 5)
    scale = 1.0 / (L + R) ** 0.5
    o_lat = mla_attention(q_t.cuda(), dev(lp), dev(lm), dev(bt), page_size, N_k, L, sl, scale=scale)
    o_full = np.einsum("bhnl,hdl->bhnd", o_lat.cpu().numpy().astype(np.float64), W_UV)
    # materialised truth: K_h = [c W_UK_h^T, rope], V_h = c W_UV_h^T, with q rounded the same way
    c_hat, rope_hat = lat_hat[..., :L], lat_hat[..., L:]
    s = np.einsum("bhnl,bgkl->bhnk", q_abs, lat_hat.astype(np.float64)) * scale
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    V_full = np.einsum("bgkl,hdl->bhkd", c_hat.astype(np.float64), W_UV)
    ref = np.einsum("bhnk,bhkd->bhnd", p, V_full)
    assert_close(o_full, ref, what="absorption identity")


@pytest.mark.parametrize("fmt", ["bf16", "e4m3"])
@pytest.mark.parametrize("DQK,DV", [(576, 512), (160, 128)])
def test_mla_bf16_and_fp8_latents_with_varlen(fmt, DQK, DV):
    """The long-context layouts: bf16 latent, and E4M3 latent with one fp32 scale per token; 128 heads,
    page 64, per-sequence context lengths, q ~ N(0,1), latent ~ N(0,1) * 0.1."""
    from fa_kernels import mla_attention
    h_q, page_size = 128, 64
    lens = [5000, 64, 4097, 1, 0, 777]
    B = len(lens)
    qdt = torch.bfloat16 if fmt == "bf16" else torch.float16
    q_t, q = randn((B, h_q, 1, DQK), 55, qdt)
    lats = [randn((1, n, DQK), 550 + i, torch.float32, 0.1)[1].astype(np.float32) for i, n in enumerate(lens)]
    if fmt == "bf16":
        stored = [torch.from_numpy(a).bfloat16() for a in lats]
        hat = [s.float().numpy() for s in stored]
        pool, bt, _ = paged_varlen([s.view(torch.int16).numpy() for s in stored], page_size, 55)
        l_pool = torch.from_numpy(pool).view(torch.bfloat16).cuda()
        scale_l = 1.0
    else:
        qs = [O.quantize_fp8_e4m3_per_token(a) for a in lats]
        hat = [O.e4m3_decode(b8) * s[..., None] for b8, s in qs]
        pool, bt, _ = paged_varlen([b8 for b8, _ in qs], page_size, 55)
        spool, bt2, _ = paged_varlen([s[..., None] for _, s in qs], page_size, 55)
        assert (bt == bt2).all()
        l_pool = dev(pool)
        scale_l = dev(spool[..., 0])                    # [num_blocks, page, 1]
    out, lse = mla_attention(q_t.cuda(), l_pool, None, dev(bt), page_size, lens, DV, scale_l, return_lse=True,
                             out_dtype=torch.float32)
    for b, n in enumerate(lens):
        if n == 0:
            assert (out[b] == 0).all() and torch.isneginf(lse[b]).all()
            continue
        ref, ref_lse = O.mla_attention_ref(q[b:b + 1], hat[b][None], DV, return_lse=True)
        tol = dict(atol=2e-3, rtol=1e-2)
        assert_close(out[b:b + 1], ref, what=f"mla {fmt} seq {b}", **tol)
        np.testing.assert_allclose(lse[b:b + 1].cpu().numpy(), ref_lse, atol=3e-3, rtol=1e-3)


def test_mla_argument_checks():
    from fa_kernels import mla_attention, mla_tc_attention
    q = torch.zeros(1, 16, 1, 96, device="cuda", dtype=torch.float16)
    lp = torch.zeros(2, 64, 1, 48, device="cuda", dtype=torch.uint8)
    lm = torch.zeros(2, 64, 1, 6, device="cuda", dtype=torch.uint8)
    bt = torch.zeros(1, 2, device="cuda", dtype=torch.int32)
    with pytest.raises(RuntimeError, match="multiple of 32"):
        mla_attention(q, lp, lm, bt, 64, 100, 48, 1.0)
    with pytest.raises(RuntimeError, match="one \\(latent\\) head"):
        mla_attention(q, lp.expand(2, 64, 2, 48), lm, bt, 64, 100, 64, 1.0)
    with pytest.raises(ValueError):
        mla_tc_attention(q, lp, lm, bt, 64, 100, 64, 1.0, engine="int4")
    with pytest.raises(RuntimeError, match="H_q>=128"):
        mla_tc_attention(q, lp, lm, bt, 64, 100, 64, 1.0, engine="nvfp4")
    with pytest.raises(RuntimeError, match="unsupported"):
        mla_attention(torch.zeros(1, 16, 1, 128, device="cuda", dtype=torch.float16),
                      torch.zeros(2, 64, 1, 64, device="cuda", dtype=torch.uint8),
                      torch.zeros(2, 64, 1, 8, device="cuda", dtype=torch.uint8), bt, 64, 100, 64, 1.0)


# ----------------------------------------------------------------- tensor-core (tcgen05) MLA path
def _bf16_latent(lens, page_size, seed, scale=0.1, DQK=576):
    lats = [randn((1, n, DQK), seed * 10 + i, torch.float32, scale)[1].astype(np.float32) for i, n in enumerate(lens)]
    stored = [torch.from_numpy(a).bfloat16() for a in lats]
    pool, bt, _ = paged_varlen([s.view(torch.int16).numpy() for s in stored], page_size, seed)
    return [s.float().numpy() for s in stored], torch.from_numpy(pool).view(torch.bfloat16).cuda(), dev(bt)


@pytest.mark.parametrize("h_q", [128, 16, 40])
@pytest.mark.parametrize("page_size", [64, 256])
def test_mla_tensor_core_path_matches_oracle_and_legacy_kernel(h_q, page_size):
    """bf16 (576, 512) latents on 64-aligned pages run on tcgen05; same inputs through the mma.sync kernel
    (engine_hint=2) and the oracle.  Lengths cover one tile, ragged tails, an empty sequence and a context
    long enough to be split (> 126 pages of 64)."""
    from fa_kernels._mla import mla_decode
    lens = [20000, 64, 4097, 1, 0, 777, 8064, 8065]
    B = len(lens)
    q_t, q = randn((B, h_q, 1, 576), 71, torch.bfloat16)
    hat, l_pool, bt = _bf16_latent(lens, page_size, 71)
    scale = 1.0 / 576 ** 0.5
    out, lse = mla_decode(q_t.cuda(), l_pool, None, bt, page_size, lens, 512, 1.0, scale, return_lse=True)
    legacy = mla_decode(q_t.cuda(), l_pool, None, bt, page_size, lens, 512, 1.0, scale, engine_hint=2)
    torch.cuda.synchronize()
    for name, o_, l_ in (("pair", out, lse),):
        for b, n in enumerate(lens):
            if n == 0:
                assert (o_[b] == 0).all() and torch.isneginf(l_[b]).all()
                continue
            ref, ref_lse = O.mla_attention_ref(q[b:b + 1], hat[b][None], 512, return_lse=True)
            assert_close(o_[b:b + 1], ref, what=f"mla tc ({name}) seq {b}")
            np.testing.assert_allclose(l_[b:b + 1].cpu().numpy(), ref_lse, atol=3e-3, rtol=1e-3)
    assert_close(out, legacy.cpu().numpy(), what="tc vs mma.sync")


def test_mla_pair_kernel_poisoned_pool_and_multi_query():
    """The CTA-pair kernel: pool slots the block table does not reference and the tail of the last page
    hold NaN (they must never reach the output), several query rows per head (rows m = h * N_q + i_q cross
    the 64-row boundary between the two CTAs), causal with q_offset, ranges split by a chunk hint."""
    from fa_kernels._mla import mla_decode
    page_size, h_q, n_q = 64, 48, 3
    lens = [700, 130, 65, 3000]
    B = len(lens)
    q_t, q = randn((B, h_q, n_q, 576), 91, torch.bfloat16)
    hat, l_pool, bt = _bf16_latent(lens, page_size, 91)
    l_pool = l_pool.clone()
    used = torch.zeros(l_pool.shape[0], dtype=torch.bool, device=l_pool.device)
    for b, n in enumerate(lens):
        npg = (n + page_size - 1) // page_size
        pages = bt[b, :npg].long()
        used[pages] = True
        if n % page_size:
            l_pool[pages[-1], n % page_size:] = float("nan")
    l_pool[~used] = float("nan")
    scale = 1.0 / 576 ** 0.5
    for causal, hint in ((False, 0), (True, 0), (True, 512)):
        q_off = [n - n_q for n in lens]
        out = mla_decode(q_t.cuda(), l_pool, None, bt, page_size, lens, 512, 1.0, scale, causal=causal,
                         q_offset=torch.tensor(q_off, dtype=torch.int32) if causal else 0, chunk_hint=hint)
        torch.cuda.synchronize()
        assert torch.isfinite(out).all()
        for b in range(B):
            ref = O.mla_attention_ref(q[b:b + 1], hat[b][None], 512, causal=causal, q_offset=q_off[b] if causal else 0)
            assert_close(out[b:b + 1], ref, what=f"mla pair causal={causal} hint={hint} seq {b}")


@pytest.mark.parametrize("causal", [False, True])
def test_mla_tensor_core_square_prefill(causal):
    from fa_kernels import mla_attention
    h_q, N, page_size = 4, 300, 64
    q_t, q = randn((2, h_q, N, 576), 72, torch.bfloat16)
    hat, l_pool, bt = _bf16_latent([N, N], page_size, 72)
    out = mla_attention(q_t.cuda(), l_pool, None, bt, page_size, N, 512, 1.0, causal=causal, q_offset=0)
    for b in range(2):
        assert_close(out[b:b + 1], O.mla_attention_ref(q[b:b + 1], hat[b][None], 512, causal=causal), what="mla tc square")
