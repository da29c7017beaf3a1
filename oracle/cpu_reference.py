"""Torch-on-CPU port of the reference's correctness anchors (TEST / BASELINE INFRASTRUCTURE only).

The reference's own CPU-capable implementation of this path is torch's scaled_dot_product_attention
wrapped by fa_kernels/reference.py; this module restates those wrappers so that the benchmark can time
"the reference's CPU path" on the host cores of a machine where the reference checkout is absent.
It is validated against the golden fixtures (tests/test_oracle_golden.py).  Nothing in the product
package imports it.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def sdpa_reference(q, k, v, *, causal=False, scale=None):
    """fa_kernels/reference.py:19-24."""
    return F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale)


def sdpa_reference_gqa(q, k, v, *, causal=False, scale=None):
    """fa_kernels/reference.py:27-43 (repeat_interleave so KV head h serves query heads [h*G, h*G+G))."""
    H_q, H_kv = q.shape[1], k.shape[1]
    if H_kv != H_q:
        assert H_q % H_kv == 0
        G = H_q // H_kv
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
    return F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale)


def sdpa_reference_mla_dequantised(q_absorbed, lat_hat, kv_lora_rank, *, causal=False, scale=None):
    """fa_kernels/reference.py:100-111 with the latent already dequantised."""
    DQK = q_absorbed.shape[-1]
    s = scale if scale is not None else 1.0 / (DQK ** 0.5)
    scores = torch.matmul(q_absorbed, lat_hat.transpose(-1, -2)) * s
    if causal:
        n_q, n_k = scores.shape[-2], scores.shape[-1]
        mask = torch.triu(torch.ones(n_q, n_k, dtype=torch.bool), diagonal=1)
        scores = scores.masked_fill(mask, float("-inf"))
    scores = scores - scores.amax(dim=-1, keepdim=True)
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, lat_hat[..., :kv_lora_rank])


def gather_dense(pool, block_table_row, page_size, n_k):
    """Dense [1, H, n_k, dx] view of one sequence of a paged pool (the gather of
    kernels/v7_paged/paged_attention.cu:118-131)."""
    n_pages = (n_k + page_size - 1) // page_size
    pages = pool[block_table_row[:n_pages].long()]                 # [n_pages, page, H, dx]
    rows = pages.reshape(n_pages * page_size, *pool.shape[2:])[:n_k]
    return rows.permute(1, 0, 2).unsqueeze(0).contiguous()
