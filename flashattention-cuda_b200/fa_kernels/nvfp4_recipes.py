"""NVFP4 scale-granularity study on the GPU — the functions of the reference's
fa_kernels/nvfp4_recipes.py (`fake_quant_nvfp4` :42, `attn_rmse` :76, `fp8_attn_rmse` :90,
`fp4_score_collapse_rmse` :105) with the quantise-dequantise steps as CUDA kernels (bit-exact with the
reference's torch code) and the attention itself through this package's dense kernel.

Granularities: "tensor" (one scale), "block16" (the stored NVFP4 format: per-16 E4M3 micro-scale +
tensor scale), "channel" (per head-dim index), "token" (per key position)."""

from __future__ import annotations

GRANULARITIES = ("tensor", "block16", "channel", "token")
_MODE = {"tensor": 0, "channel": 1, "token": 2}


def fake_quant_nvfp4(x, granularity: str = "block16", *, e4m3_scale: bool = True):
    """Quantise `x` to NVFP4 levels at `granularity` and return the dequantised tensor (x's shape and dtype)."""
    import ctypes as C

    import torch

    from . import _lib
    from ._formats import dequantize_nvfp4, quantize_nvfp4
    if granularity == "block16":
        p, m, s = quantize_nvfp4(x)
        return dequantize_nvfp4(p, m, s).to(x.dtype)
    if granularity not in _MODE:
        raise ValueError(f"unknown granularity {granularity!r}; pick one of {GRANULARITIES}")
    if not x.is_cuda:
        raise RuntimeError("fake_quant_nvfp4 runs on the GPU: pass a CUDA tensor")
    lib = _lib.load()
    xf = x.float().contiguous()
    d = xf.shape[-1]
    rows = xf.numel() // d
    out = torch.empty_like(xf)
    scratch = torch.empty(max(rows, d, 1), dtype=torch.int32, device=x.device)
    lib.fa_fake_quant_e2m1.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                       C.c_size_t, C.c_void_p]
    with torch.cuda.device(x.device):
        _lib.check(lib.fa_fake_quant_e2m1(xf.data_ptr(), rows, d, _MODE[granularity], int(bool(e4m3_scale)), out.data_ptr(),
                                          scratch.data_ptr(), scratch.numel() * 4,
                                          torch.cuda.current_stream(x.device).cuda_stream), "fa_fake_quant_e2m1")
    return out.to(x.dtype)


def _gqa_attention(q, k, v, causal=False):
    """Dense GQA attention through the tensor-core kernel (KV heads expanded, reference.py:27-43)."""
    from . import attention
    G = q.shape[1] // k.shape[1]
    if G > 1:
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
    return attention(q, k, v, causal=causal)


def _rmse(a, b):
    return (a.float() - b.float()).pow(2).mean().sqrt().item()


def attn_rmse(q, k, v, *, k_gran: str, v_gran: str, causal: bool = False) -> float:
    """End-to-end attention RMSE of (K quantised at k_gran, V at v_gran) against unquantised KV."""
    out_q = _gqa_attention(q, fake_quant_nvfp4(k, k_gran), fake_quant_nvfp4(v, v_gran), causal)
    return _rmse(out_q, _gqa_attention(q, k, v, causal))


def fp8_attn_rmse(q, k, v, *, causal: bool = False) -> float:
    """The FP8 floor: K, V per-tensor E4M3."""
    from ._formats import dequantize_fp8_e4m3, quantize_fp8_e4m3
    kq = dequantize_fp8_e4m3(*quantize_fp8_e4m3(k)).to(k.dtype)
    vq = dequantize_fp8_e4m3(*quantize_fp8_e4m3(v)).to(v.dtype)
    return _rmse(_gqa_attention(q, kq, vq, causal), _gqa_attention(q, k, v, causal))


def fp4_score_collapse_rmse(q, k, v, *, causal: bool = False) -> dict:
    """FP4 for the softmax weights as well as for the KV cache (reference nvfp4_recipes.py:105-142):
    output RMSE against exact attention of (a) "fp4_kv_only": K quantised per channel, V per token, exact
    weights; (b) "fp4_kv_and_p": the same with the weights P quantised per query row and renormalised.

    This is the one function of the study that needs the weights themselves, which no attention kernel
    materialises: as in the reference, the [N_q, N_k] score matrix is built with plain fp32 matrix
    products (torch, on the GPU); every quantisation step runs through this library's kernels."""
    import torch

    G = q.shape[1] // k.shape[1]

    def expand(x):
        return x.repeat_interleave(G, dim=1).float() if G > 1 else x.float()

    qf = q.float()
    scale = 1.0 / (q.shape[-1] ** 0.5)
    mask = None
    if causal:
        mask = torch.triu(torch.ones(q.shape[-2], k.shape[-2], device=q.device, dtype=torch.bool), diagonal=1)

    def weights(keys):
        s = torch.matmul(qf, keys.transpose(-1, -2)) * scale
        if mask is not None:
            s = s.masked_fill(mask, float("-inf"))
        return torch.softmax(s, dim=-1)

    ve = expand(v)
    out_ref = torch.matmul(weights(expand(k)), ve)
    vq = expand(fake_quant_nvfp4(v, "token"))
    p_kv = weights(expand(fake_quant_nvfp4(k, "channel")))
    out_kv = torch.matmul(p_kv, vq)
    p_q = fake_quant_nvfp4(p_kv, "token")
    p_q = p_q / p_q.sum(dim=-1, keepdim=True).clamp_min(1e-12)
    out_pq = torch.matmul(p_q, vq)
    return {"fp4_kv_only": _rmse(out_kv, out_ref), "fp4_kv_and_p": _rmse(out_pq, out_ref)}
