"""The numpy oracle against fixtures produced by the reference's own Python code (CPU only).

Integer / byte work must agree bit-for-bit; float attention outputs to 1e-5 (the reference runs
torch SDPA in fp32, the oracle runs in fp64).
"""

from __future__ import annotations

import numpy as np

from oracle import fa_oracle as O


def test_e4m3_decode_all_bytes(golden):
    g = golden("e4m3_codec.npz")
    mine = O.e4m3_decode(np.arange(256, dtype=np.uint8))
    np.testing.assert_array_equal(np.isnan(mine), np.isnan(g["decoded"]))
    ok = ~np.isnan(mine)
    np.testing.assert_array_equal(mine[ok], g["decoded"][ok])


def test_e4m3_encode_probes_bit_exact(golden):
    g = golden("e4m3_codec.npz")
    mine = O.e4m3_encode(g["probes"])
    np.testing.assert_array_equal(mine, g["encoded"])


def test_quantize_fp8_bit_exact(golden):
    g = golden("quant_fp8.npz")
    b, s = O.quantize_fp8_e4m3(g["x"])
    assert s == float(g["scale"])
    np.testing.assert_array_equal(b, g["bytes"])
    np.testing.assert_array_equal(O.dequantize_fp8_e4m3(b, s), g["dequant"])


def test_quantize_fp8_per_token_matches_per_tensor_formula(golden):
    g = golden("quant_fp8.npz")
    x = g["x"]
    b, s = O.quantize_fp8_e4m3_per_token(x)
    assert s.shape == x.shape[:-1]
    # each (token, head) row must equal the per-tensor quantiser applied to that row alone
    for idx in [(0, 0, 0), (0, 1, 7), (1, 0, 39)]:
        rb, rs = O.quantize_fp8_e4m3(x[idx])
        assert np.float32(rs) == s[idx]
        np.testing.assert_array_equal(rb, b[idx])


def test_quantize_nvfp4_bit_exact(golden):
    g = golden("quant_nvfp4.npz")
    p, m, s = O.quantize_nvfp4(g["x"])
    assert s == float(g["scale"])
    np.testing.assert_array_equal(m, g["micro"])
    np.testing.assert_array_equal(p, g["packed"])
    np.testing.assert_array_equal(O.dequantize_nvfp4(p, m, s), g["dequant"])
    # documented edge semantics: the all-zero block has micro byte 0 and 0x77 nibble bytes
    assert (g["micro"][0, 0, 3, 1] == 0) and (g["packed"][0, 0, 3, 8:16] == 0x77).all()


def test_pager_bit_exact(golden):
    g = golden("paged.npz")
    perm = g["block_table"].reshape(-1)
    kp, vp, bt, nk = O.build_paged_kv(g["k"], g["v"], int(g["page_size"]), perm)
    np.testing.assert_array_equal(kp, g["k_pool"])
    np.testing.assert_array_equal(vp, g["v_pool"])
    np.testing.assert_array_equal(bt, g["block_table"])
    # gather through the table returns the dense rows
    for b in range(2):
        rows = O.paged_gather(kp, bt[b], int(g["page_size"]), nk)
        np.testing.assert_array_equal(rows, g["k"][b])


def test_sdpa_oracles(golden):
    g = golden("sdpa.npz")
    q, k, v = g["q"], g["k"], g["v"]
    tol = dict(atol=1e-5, rtol=1e-5)
    np.testing.assert_allclose(O.attention_ref(q, k, v), g["out"], **tol)
    np.testing.assert_allclose(O.attention_ref(q, k, v, causal=True), g["out_causal"], **tol)
    np.testing.assert_allclose(O.attention_ref(q, k, v, scale=0.1), g["out_scale"], **tol)
    np.testing.assert_allclose(O.attention_ref(q, k, v, causal=True), g["out_fp64"], **tol)
    np.testing.assert_allclose(O.gqa_attention_ref(q, g["kg"], g["vg"]), g["out_gqa"], **tol)
    np.testing.assert_allclose(O.gqa_attention_ref(q, g["kg"], g["vg"], causal=True), g["out_gqa_causal"], **tol)
    np.testing.assert_allclose(O.gqa_attention_ref(g["qd"], g["kg"], g["vg"]), g["out_gqa_decode"], **tol)


def test_lse_is_consistent_with_output(golden):
    g = golden("sdpa.npz")
    q, k, v = g["q"].astype(np.float64), g["k"].astype(np.float64), g["v"].astype(np.float64)
    out, lse = O.attention_ref(q, k, v, causal=True, return_lse=True)
    s = np.matmul(q, np.swapaxes(k, -1, -2)) / 8.0
    s = np.where(np.triu(np.ones((48, 48), bool), 1), -np.inf, s)
    np.testing.assert_allclose(lse, np.log(np.exp(s).sum(-1)), rtol=1e-12)


def test_quantised_kv_oracles(golden):
    g = golden("quant_attn.npz")
    q, k, v = g["q"], g["k"], g["v"]
    kb, sk = O.quantize_fp8_e4m3(k)
    vb, sv = O.quantize_fp8_e4m3(v)
    assert sk == float(g["sk"]) and sv == float(g["sv"])
    out = O.gqa_attention_ref(q, O.dequantize_fp8_e4m3(kb, sk), O.dequantize_fp8_e4m3(vb, sv))
    np.testing.assert_allclose(out, g["out_fp8"], atol=1e-5, rtol=1e-5)
    out4 = O.gqa_attention_ref(q, O.dequantize_nvfp4(*O.quantize_nvfp4(k)), O.dequantize_nvfp4(*O.quantize_nvfp4(v)))
    np.testing.assert_allclose(out4, g["out_nvfp4"], atol=1e-5, rtol=1e-5)


def test_mla_oracles(golden):
    g = golden("mla.npz")
    L = int(g["kv_lora_rank"])
    lat_hat = O.dequantize_nvfp4(*O.quantize_nvfp4(g["latent"]))
    np.testing.assert_array_equal(lat_hat, g["lat_hat"])
    np.testing.assert_allclose(O.mla_attention_ref(g["q"], lat_hat, L), g["out"], atol=1e-5, rtol=1e-5)
    np.testing.assert_allclose(O.mla_attention_ref(g["q_square"], lat_hat, L, causal=True),
                               g["out_square_causal"], atol=1e-5, rtol=1e-5)
    # absorption identity (reference.py:114-145): absorbed kernel output re-projected through W_UV
    q_abs = np.concatenate([np.einsum("bhnd,hdl->bhnl", g["q_nope"], g["W_UK"]), g["q_rope"]], -1)
    o_lat = O.mla_attention_ref(q_abs, lat_hat, L, scale=1.0 / (96 ** 0.5))
    o_full = np.einsum("bhnl,hdl->bhnd", o_lat, g["W_UV"])
    np.testing.assert_allclose(o_full, g["out_materialized"], atol=2e-5, rtol=1e-4)


def test_merge_of_key_ranges_equals_full(golden):
    g = golden("sdpa.npz")
    q, k, v = g["qd"], g["kg"], g["vg"]
    full, lse_full = O.gqa_attention_ref(q, k, v, return_lse=True)
    parts = [O.gqa_attention_ref(q, k[:, :, a:b], v[:, :, a:b], return_lse=True)
             for a, b in [(0, 7), (7, 7), (7, 30), (30, 48)] if True]
    # an empty range contributes zeros with LSE = -inf
    o = np.stack([p[0] if p[0].size else np.zeros_like(full) for p in parts])
    l = np.stack([p[1] if p[1].size else np.full_like(lse_full, -np.inf) for p in parts])
    merged, lse = O.merge_partials_ref(o, l)
    np.testing.assert_allclose(merged, full, atol=1e-12)
    np.testing.assert_allclose(lse, lse_full, atol=1e-12)


def test_nvfp4_recipes(golden):
    g = golden("recipes.npz")
    q, k, v = g["q"], g["k"], g["v"]
    for gran in ("tensor", "block16", "channel", "token"):
        np.testing.assert_array_equal(O.fake_quant_nvfp4(k, gran), g[f"fq_k_{gran}"])
        np.testing.assert_array_equal(O.fake_quant_nvfp4(k, gran, e4m3_scale=False), g[f"fq_k_{gran}_fp32scale"])
    np.testing.assert_allclose(O.attn_rmse(q, k, v, k_gran="block16", v_gran="block16"),
                               float(g["rmse_block_block"]), rtol=1e-4)
    np.testing.assert_allclose(O.attn_rmse(q, k, v, k_gran="channel", v_gran="token"),
                               float(g["rmse_channel_token"]), rtol=1e-4)
    np.testing.assert_allclose(O.fp8_attn_rmse(q, k, v), float(g["rmse_fp8"]), rtol=1e-4)
    col = O.fp4_score_collapse_rmse(q, k, v)
    np.testing.assert_allclose(col["fp4_kv_only"], float(g["collapse_kv_only"]), rtol=1e-4)
    np.testing.assert_allclose(col["fp4_kv_and_p"], float(g["collapse_kv_and_p"]), rtol=1e-3)


def test_config1_cpu_plumbing(golden):
    """Dense causal MHA, B=2 H=8 N=512 d=64 fp32 from seed 0 (the reference's CPU-runnable case)."""
    import torch
    g = golden("config1_sample.npz")
    torch.manual_seed(0)
    q = torch.randn(2, 8, 512, 64)
    k = torch.randn(2, 8, 512, 64)
    v = torch.randn(2, 8, 512, 64)
    stride = int(g["stride"])
    np.testing.assert_array_equal(q.flatten()[::stride].numpy(), g["q_sample"])   # generator unchanged
    out, lse = O.attention_ref(q.numpy(), k.numpy(), v.numpy(), causal=True, scale=0.125, return_lse=True)
    np.testing.assert_allclose(out.reshape(-1)[::stride], g["out_sample"], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(np.abs(out).sum(), float(g["out_abs_sum"]), rtol=1e-6)
    assert lse.shape == (2, 8, 512) and np.isfinite(lse).all()


def test_torch_cpu_port_matches_reference_outputs(golden):
    import torch
    from oracle import cpu_reference as R
    g = golden("sdpa.npz")
    t = lambda a: torch.from_numpy(a)
    np.testing.assert_allclose(R.sdpa_reference(t(g["q"]), t(g["k"]), t(g["v"]), causal=True).numpy(),
                               g["out_causal"], atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(R.sdpa_reference_gqa(t(g["qd"]), t(g["kg"]), t(g["vg"])).numpy(),
                               g["out_gqa_decode"], atol=1e-6, rtol=1e-6)
    m = golden("mla.npz")
    np.testing.assert_allclose(
        R.sdpa_reference_mla_dequantised(t(m["q"]), t(m["lat_hat"]), int(m["kv_lora_rank"])).numpy(),
        m["out"], atol=1e-6, rtol=1e-6)
    p = golden("paged.npz")
    dense = R.gather_dense(t(p["k_pool"]), t(p["block_table"])[1], int(p["page_size"]), int(p["n_k"]))
    np.testing.assert_array_equal(dense[0].numpy(), p["k"][1])
