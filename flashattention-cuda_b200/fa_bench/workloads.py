"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark
configurations.  Everything is generated on the device; the KV of a paged workload is drawn directly
into the pool (for i.i.d. values that equals scattering a dense draw) and the block table is a random
permutation of the physical pages."""

from __future__ import annotations

import torch


def paged_gqa_decode(device, *, batch=64, h_q=32, h_kv=8, d=128, page_size=16, min_len=1024, max_len=8192,
                     seed=2, kv_dtype=torch.float16, seq_lens=None, data_seed=None):
    """Paged GQA decode: one query token per sequence, context lengths uniform in [min_len, max_len],
    block table = random permutation of the physical pages, K/V ~ N(0,1).  `seed` draws the lengths and
    the page permutation, `data_seed` (default: `seed`) the tensor values.

    Returns a dict with q, k_pool, v_pool, block_table, page_size, seq_lens (python list) and the
    algorithmic byte counts.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    if seq_lens is None:
        seq_lens = torch.randint(min_len, max_len + 1, (batch,), generator=g).tolist()
    batch = len(seq_lens)
    n_pages = [(n + page_size - 1) // page_size for n in seq_lens]
    total_pages = sum(n_pages)
    n_logical = max(n_pages)
    perm = torch.randperm(total_pages, generator=g)
    bt = torch.zeros(batch, n_logical, dtype=torch.int32)
    cur = 0
    for b, np_ in enumerate(n_pages):
        bt[b, :np_] = perm[cur:cur + np_].to(torch.int32)
        cur += np_
    gd = torch.Generator(device=device).manual_seed(seed if data_seed is None else data_seed)
    k_pool = torch.randn(total_pages, page_size, h_kv, d, device=device, dtype=torch.float32, generator=gd).to(kv_dtype)
    v_pool = torch.randn(total_pages, page_size, h_kv, d, device=device, dtype=torch.float32, generator=gd).to(kv_dtype)
    q = torch.randn(batch, h_q, 1, d, device=device, dtype=torch.float32, generator=gd).to(kv_dtype)
    tokens = sum(seq_lens)
    esz = k_pool.element_size()
    kv_bytes = tokens * 2 * h_kv * d * esz
    other = 2 * q.numel() * esz + 4 * total_pages
    return dict(q=q, k_pool=k_pool, v_pool=v_pool, block_table=bt.to(device), block_table_host=bt,
                page_size=page_size, seq_lens=seq_lens, tokens=tokens, kv_bytes=kv_bytes,
                total_bytes=kv_bytes + other, flops=4 * h_q * d * tokens)


def causal_prefill(device, *, batch=4, heads=32, n=4096, d=128, seed=1, dtype=torch.float16):
    """Dense causal prefill: q, k, v ~ N(0,1) * 0.5 from `seed`, [batch, heads, n, d]."""
    g = torch.Generator(device=device).manual_seed(seed)
    shape = (batch, heads, n, d)
    q, k, v = ((torch.randn(shape, device=device, generator=g) * 0.5).to(dtype) for _ in range(3))
    flops_causal = 2 * batch * heads * d * n * (n + 1)          # both matmuls, lower triangle only
    return dict(q=q, k=k, v=v, flops=flops_causal, flops_full=4 * batch * heads * n * n * d,
                bytes=4 * q.numel() * q.element_size())


def mla_decode(device, *, batch=128, h_q=128, dqk=576, dv=512, page_size=64, min_len=4096, max_len=32768, seed=5,
               latent="bf16", seq_lens=None):
    """MLA latent decode (DeepSeek-V3-like): q ~ N(0,1), latent ~ N(0,1) * 0.1 drawn straight into the
    paged pool, context lengths uniform in [min_len, max_len]; latent stored as bf16 or as E4M3 bytes
    with one fp32 scale per token (scale = amax / 448)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    if seq_lens is None:
        seq_lens = torch.randint(min_len, max_len + 1, (batch,), generator=g).tolist()
    batch = len(seq_lens)
    n_pages = [(n + page_size - 1) // page_size for n in seq_lens]
    total_pages = sum(n_pages)
    perm = torch.randperm(total_pages, generator=g)
    bt = torch.zeros(batch, max(n_pages), dtype=torch.int32)
    cur = 0
    for b, np_ in enumerate(n_pages):
        bt[b, :np_] = perm[cur:cur + np_].to(torch.int32)
        cur += np_
    gd = torch.Generator(device=device).manual_seed(seed)
    pool = torch.empty(total_pages, page_size, 1, dqk, device=device, dtype=torch.bfloat16)
    step = 4096
    for i in range(0, total_pages, step):                      # generate in slabs to bound fp32 temporaries
        n = min(step, total_pages - i)
        pool[i:i + n] = (torch.randn(n, page_size, 1, dqk, device=device, generator=gd) * 0.1).to(torch.bfloat16)
    q = torch.randn(batch, h_q, 1, dqk, device=device, generator=gd)
    tokens = sum(seq_lens)
    out = dict(block_table=bt.to(device), block_table_host=bt, page_size=page_size, seq_lens=seq_lens, tokens=tokens,
               kv_lora_rank=dv, flops=2 * h_q * (dqk + dv) * tokens)
    if latent == "bf16":
        out.update(q=q.to(torch.bfloat16), l_pool=pool, scale_l=1.0, latent_bytes=tokens * dqk * 2)
    elif latent == "e4m3":
        from fa_kernels.paged import quantize_fp8_e4m3_per_token
        bytes_, scales = quantize_fp8_e4m3_per_token(pool)
        out.update(q=q.to(torch.float16), l_pool=bytes_, scale_l=scales, latent_bytes=tokens * (dqk + 4))
    else:
        raise ValueError(latent)
    return out


def quantised_long_context_decode(device, *, fmt="e4m3", batch=4, h_q=32, h_kv=8, d=128, ctx=1048576, page_size=64, seed=3):
    """Quantised-KV long-context GQA decode: K, V ~ N(0,1) with a fixed random 1 % of the channels
    (per KV head) scaled x10, quantised (a) "e4m3": FP8 with one fp32 scale per token per head =
    amax / 448, or (b) "nvfp4": E2M1 + one E4M3 scale per 16 elements + one fp32 tensor scale; paged
    with a shuffled block table.  Built sequence by sequence to bound the fp32 temporaries."""
    from fa_kernels import paged as P
    gd = torch.Generator(device=device).manual_seed(seed)
    n_out = max(1, round(0.01 * d))
    chan = torch.ones(1, h_kv, 1, d, device=device)
    for h in range(h_kv):
        idx = torch.randperm(d, device=device, generator=gd)[:n_out]
        chan[0, h, 0, idx] = 10.0
    k = torch.empty(batch, h_kv, ctx, d, device=device, dtype=torch.float16)
    v = torch.empty(batch, h_kv, ctx, d, device=device, dtype=torch.float16)
    for b in range(batch):
        k[b] = (torch.randn(1, h_kv, ctx, d, device=device, generator=gd) * chan)[0].half()
        v[b] = (torch.randn(1, h_kv, ctx, d, device=device, generator=gd) * chan)[0].half()
    q = torch.randn(batch, h_q, 1, d, device=device, generator=gd).half()
    tokens = batch * ctx
    w = dict(q=q, page_size=page_size, n_k=ctx, tokens=tokens, fmt=fmt, flops=4 * h_q * d * tokens)
    if fmt == "e4m3":
        kp, vp, bt, _, ks, vs = P.build_paged_kv_fp8_per_token(k, v, page_size, seed=seed)
        w.update(k_pool=kp, v_pool=vp, block_table=bt, k_scale=ks, v_scale=vs, kv_bytes=2 * h_kv * tokens * (d + 4))
    elif fmt == "nvfp4":
        kp, km, vp, vm, bt, _, sk, sv = P.build_paged_kv_nvfp4(k, v, page_size, seed=seed)
        w.update(k_pool=kp, k_micro=km, v_pool=vp, v_micro=vm, block_table=bt, k_scale=sk, v_scale=sv,
                 kv_bytes=2 * h_kv * tokens * (d // 2 + d // 16))
    else:
        raise ValueError(fmt)
    del k, v
    return w
