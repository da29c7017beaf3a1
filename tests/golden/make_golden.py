"""Generate the golden fixtures in this directory from the reference project's own Python code.

Run once in a container that has the reference checkout (it cannot travel to the GPU machine):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `fa_kernels` package read-only (its oracles and quantisers run on CPU),
feeds it small seeded inputs, and stores inputs + outputs as compressed .npz files.  The tests then
check the numpy oracle (oracle/fa_oracle.py) and the CUDA kernels against these files without the
reference being present.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from fa_kernels import nvfp4_recipes, paged, reference  # noqa: E402  (the reference's own modules)

    def save(name, **arrs):
        np.savez_compressed(os.path.join(HERE, name), **{k: np.asarray(v) for k, v in arrs.items()})

    # ---- E4M3 codec: all 256 bytes decoded, and a probe set encoded (ties, range edges, subnormals)
    all_bytes = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    decoded = all_bytes.view(torch.float8_e4m3fn).float()
    g = torch.Generator().manual_seed(11)
    probes = torch.cat([
        torch.randn(4096, generator=g) * 100.0,
        torch.randn(4096, generator=g),
        torch.randn(2048, generator=g) * 0.01,
        torch.tensor([0.0, -0.0, 448.0, -448.0, 456.0, 463.9, 464.0, 447.9, 2.0 ** -9, 2.0 ** -10,
                      1.5 * 2.0 ** -10, 3.0 * 2.0 ** -10, 2.0 ** -6, 0.0175, 1.0625, 1.1875, 17.0, 19.0]),
        # every midpoint between adjacent representable magnitudes (the RNE tie cases)
        (decoded[:126] + decoded[1:127]) / 2,
    ])
    enc = probes.to(torch.float8_e4m3fn).view(torch.uint8)
    save("e4m3_codec.npz", decoded=decoded.numpy(), probes=probes.numpy(), encoded=enc.numpy())

    # ---- per-tensor FP8 quantiser
    torch.manual_seed(21)
    x = torch.randn(2, 2, 40, 64) * 3.0
    x[0, 0, 0, :8] = 0.0
    b8, s8 = paged.quantize_fp8_e4m3(x)
    save("quant_fp8.npz", x=x.numpy(), bytes=b8.numpy(), scale=np.float64(s8),
         dequant=paged.dequantize_fp8_e4m3(b8, s8).numpy())

    # ---- NVFP4 quantiser incl. an all-zero block, a negative zero, and engineered rounding ties
    torch.manual_seed(22)
    x = torch.randn(1, 2, 24, 64)
    x[0, 0, 3, 16:32] = 0.0            # all-zero 16-block inside a non-zero tensor
    x[0, 1, 5, 0] = -0.0
    x[0, 0, 0, 0] = 6.0                # pins the tensor amax so block 0 of token 0 has micro = exact
    x[0, 0, 0, 1:8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])   # exact midpoints
    x[0, 0, 0, 8:15] = -torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    pk, mi, s4 = paged.quantize_nvfp4(x)
    save("quant_nvfp4.npz", x=x.numpy(), packed=pk.numpy(), micro=mi.numpy(), scale=np.float64(s4),
         dequant=paged.dequantize_nvfp4(pk, mi, s4).numpy())

    # ---- pager (CPU generator)
    torch.manual_seed(23)
    k = torch.randn(2, 2, 37, 16)
    v = torch.randn(2, 2, 37, 16)
    kp, vp, bt, nk = paged.build_paged_kv(k, v, 8, seed=6)
    save("paged.npz", k=k.numpy(), v=v.numpy(), k_pool=kp.numpy(), v_pool=vp.numpy(),
         block_table=bt.numpy(), n_k=nk, page_size=8)

    # ---- dense + GQA SDPA oracles
    torch.manual_seed(24)
    q = torch.randn(1, 4, 48, 64)
    k = torch.randn(1, 4, 48, 64)
    v = torch.randn(1, 4, 48, 64)
    kg = torch.randn(1, 2, 48, 64)
    vg = torch.randn(1, 2, 48, 64)
    qd = torch.randn(1, 4, 1, 64)
    save("sdpa.npz", q=q.numpy(), k=k.numpy(), v=v.numpy(), kg=kg.numpy(), vg=vg.numpy(), qd=qd.numpy(),
         out=reference.sdpa_reference(q, k, v).numpy(),
         out_causal=reference.sdpa_reference(q, k, v, causal=True).numpy(),
         out_scale=reference.sdpa_reference(q, k, v, scale=0.1).numpy(),
         out_gqa=reference.sdpa_reference_gqa(q, kg, vg).numpy(),
         out_gqa_causal=reference.sdpa_reference_gqa(q, kg, vg, causal=True).numpy(),
         out_gqa_decode=reference.sdpa_reference_gqa(qd, kg, vg).numpy(),
         out_fp64=reference.fp64_reference(q, k, v, causal=True).numpy())

    # ---- quantised-KV apples-to-apples oracles
    torch.manual_seed(25)
    q = torch.randn(1, 4, 1, 64)
    k = torch.randn(1, 2, 96, 64)
    v = torch.randn(1, 2, 96, 64)
    _, sk = paged.quantize_fp8_e4m3(k)
    _, sv = paged.quantize_fp8_e4m3(v)
    save("quant_attn.npz", q=q.numpy(), k=k.numpy(), v=v.numpy(), sk=np.float64(sk), sv=np.float64(sv),
         out_fp8=reference.sdpa_reference_gqa_fp8(q, k, v, sk, sv).numpy(),
         out_nvfp4=reference.sdpa_reference_gqa_nvfp4(q, k, v).numpy())

    # ---- MLA oracles (small latent: DQK = 96, DV = 64)
    torch.manual_seed(26)
    h_q, L, R, n = 8, 64, 32, 80
    qa = torch.randn(1, h_q, 1, L + R)
    lat = torch.randn(1, 1, n, L + R)
    qsq = torch.randn(1, h_q, n, L + R)
    Dn, Dv = 48, 40
    q_nope = torch.randn(1, h_q, 1, Dn)
    q_rope = torch.randn(1, h_q, 1, R)
    W_UK = torch.randn(h_q, Dn, L) / (L ** 0.5)
    W_UV = torch.randn(h_q, Dv, L) / (L ** 0.5)
    lp, lm, sl = paged.quantize_nvfp4(lat)
    save("mla.npz", q=qa.numpy(), latent=lat.numpy(), q_square=qsq.numpy(), kv_lora_rank=L,
         lat_hat=paged.dequantize_nvfp4(lp, lm, sl).numpy(),
         out=reference.sdpa_reference_mla(qa, lat, L).numpy(),
         out_square_causal=reference.sdpa_reference_mla(qsq, lat, L, causal=True).numpy(),
         q_nope=q_nope.numpy(), q_rope=q_rope.numpy(), W_UK=W_UK.numpy(), W_UV=W_UV.numpy(),
         out_materialized=reference.sdpa_reference_mla_materialized(
             q_nope, q_rope, lat, L, W_UK, W_UV, scale=1.0 / ((L + R) ** 0.5)).numpy())

    # ---- NVFP4 recipe study
    torch.manual_seed(27)
    q = torch.randn(1, 4, 8, 32)
    k = torch.randn(1, 2, 64, 32)
    v = torch.randn(1, 2, 64, 32)
    k[..., 5] *= 10.0                  # an outlier channel
    v[:, :, 7, :] *= 10.0              # an outlier token
    rec = {"q": q.numpy(), "k": k.numpy(), "v": v.numpy()}
    for gname in nvfp4_recipes.GRANULARITIES:
        rec[f"fq_k_{gname}"] = nvfp4_recipes.fake_quant_nvfp4(k, gname).numpy()
        rec[f"fq_k_{gname}_fp32scale"] = nvfp4_recipes.fake_quant_nvfp4(k, gname, e4m3_scale=False).numpy()
    rec["rmse_block_block"] = nvfp4_recipes.attn_rmse(q, k, v, k_gran="block16", v_gran="block16")
    rec["rmse_channel_token"] = nvfp4_recipes.attn_rmse(q, k, v, k_gran="channel", v_gran="token")
    rec["rmse_fp8"] = nvfp4_recipes.fp8_attn_rmse(q, k, v)
    col = nvfp4_recipes.fp4_score_collapse_rmse(q, k, v)
    rec["collapse_kv_only"] = col["fp4_kv_only"]
    rec["collapse_kv_and_p"] = col["fp4_kv_and_p"]
    save("recipes.npz", **rec)

    # ---- the CPU plumbing configuration: dense causal MHA, B=2 H=8 N=512 d=64, fp32, seed 0.
    # Inputs are regenerated from the seed by the tests (a strided input sample is stored to detect
    # generator drift); the output is stored as a strided sample to keep the fixture small.
    torch.manual_seed(0)
    q = torch.randn(2, 8, 512, 64)
    k = torch.randn(2, 8, 512, 64)
    v = torch.randn(2, 8, 512, 64)
    out = reference.sdpa_reference(q, k, v, causal=True, scale=0.125)
    stride = 61
    save("config1_sample.npz", stride=stride, q_sample=q.flatten()[::stride].numpy(),
         out_sample=out.flatten()[::stride].numpy(),
         out_abs_sum=np.float64(out.double().abs().sum().item()))

    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
