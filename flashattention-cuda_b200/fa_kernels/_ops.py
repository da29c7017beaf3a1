"""The `forward` of each operator family with the reference's positional signatures
(kernels/*/binding.cpp) plus keyword-only extensions (`out_dtype`, `return_lse`, per-sequence
lengths through `n_k`, per-token FP8 scales through tensor-valued `scale_k` / `scale_v`)."""

from __future__ import annotations

import torch

from . import _decode


def paged_forward(q, k_pool, v_pool, block_table, page_size, n_k, scale, causal=False, q_offset=0, **kw):
    """kernels/v7_paged/binding.cpp, kernels/v8_gqa_ss/binding.cpp:9-20."""
    return _decode.paged_decode(q, k_pool, v_pool, block_table, page_size, n_k, scale, causal, q_offset,
                                kv_format="bf16" if k_pool.dtype == torch.bfloat16 else "f16", **kw)


def fp8_forward(q, k_pool, v_pool, block_table, page_size, n_k, scale_k, scale_v, scale, causal=False,
                q_offset=0, **kw):
    """kernels/v9_fp8/binding.cpp:9-23.  `scale_k` / `scale_v` are floats (per tensor, the reference
    layout) or float32 tensors [num_blocks, page_size, H_kv] (one scale per token per head)."""
    if isinstance(scale_k, torch.Tensor) and scale_k.numel() > 1:
        return _decode.paged_decode(q, k_pool, v_pool, block_table, page_size, n_k, scale, causal, q_offset,
                                    kv_format="e4m3", k_token_scale=scale_k, v_token_scale=scale_v, **kw)
    return _decode.paged_decode(q, k_pool, v_pool, block_table, page_size, n_k, scale, causal, q_offset,
                                kv_format="e4m3", scale_k=float(scale_k), scale_v=float(scale_v), **kw)


def nvfp4_forward(q, k_pool, k_scale, v_pool, v_scale, block_table, page_size, n_k, scale_k, scale_v, scale,
                  causal=False, q_offset=0, **kw):
    """kernels/v10_nvfp4/binding.cpp."""
    return _decode.paged_decode(q, k_pool, v_pool, block_table, page_size, n_k, scale, causal, q_offset,
                                kv_format="nvfp4", k_micro=k_scale, v_micro=v_scale,
                                scale_k=float(scale_k), scale_v=float(scale_v), **kw)


def dense_forward(q, k, v, scale, causal, **kw):
    """kernels/v1_naive/binding.cpp:7-14 (same signature in v2..v6)."""
    from . import _dense
    return _dense.dense_attention(q, k, v, scale, causal, **kw)


def mla_forward(q, l_pool, l_scale, block_table, page_size, n_k, kv_lora_rank, scale_l, scale, causal=False,
                q_offset=0, **kw):
    """kernels/v11_mla/binding.cpp.  `l_pool` may also be a bf16 latent [.., 1, DQK] or an FP8 E4M3
    latent (uint8 [.., 1, DQK]; `scale_l` then a float or per-token float32 scales); `l_scale` (the
    NVFP4 micro-scale pool) is ignored for those."""
    from . import _mla
    return _mla.mla_decode(q, l_pool, l_scale, block_table, page_size, n_k, kv_lora_rank, scale_l, scale, causal,
                           q_offset, **kw)


def mla_tc_forward(q, l_pool, l_scale, block_table, page_size, n_k, kv_lora_rank, scale_l, scale, causal=False,
                   q_offset=0, engine=0, **kw):
    """kernels/v12_mla_tc/binding.cpp:11-27.  The reference validates and then raises (it ships no device
    code for this backend); here both engines run the tensor-core MLA kernel.  The engine-1 gate of the
    reference (H_q >= 128, mla_tc_attention.cu:119-123) and the engine-0 gate (H_q >= 16) are kept."""
    if engine not in (0, 1):
        raise RuntimeError(f"engine must be 0 (FP8 Arm 1) or 1 (NVFP4 Arm 2); got {engine}")
    H_q = q.shape[1]
    if engine == 1 and H_q < 128:
        raise RuntimeError(f"v12 Arm 2 (native NVFP4 MMA) needs M=H_q>=128; got H_q={H_q} — use engine=0 (FP8) below 128")
    if engine == 0 and H_q < 16:
        raise RuntimeError(f"v12 Arm 1 (FP8 MMA) packs M=H_q; got H_q={H_q}")
    return mla_forward(q, l_pool, l_scale, block_table, page_size, n_k, kv_lora_rank, scale_l, scale, causal,
                       q_offset, **kw)
