"""KV-cache formats and paged layout builders on the GPU (kernels of csrc/quant.cu).

Same names, arguments and return values as the reference's torch helpers in fa_kernels/paged.py
(`quantize_fp8_e4m3` :94, `dequantize_fp8_e4m3` :112, `quantize_nvfp4` :136, `dequantize_nvfp4` :173,
`build_paged_kv` :48, `build_paged_kv_fp8` :121, `build_paged_kv_nvfp4` :192, `build_paged_kv_mla`
:287) and byte-identical results.  Inputs must be CUDA tensors; torch supplies memory and the random
permutation only.
"""

from __future__ import annotations

import torch

from . import _lib
from ._lib import FA_BF16, FA_F16, FA_F32

_DT = {torch.float32: FA_F32, torch.float16: FA_F16, torch.bfloat16: FA_BF16}


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _src(x):
    _require(x.is_cuda, "quantisers and pagers run on the GPU: pass CUDA tensors")
    if x.dtype not in _DT:
        x = x.float()
    return x.contiguous()


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def quantize_fp8_e4m3(x):
    """Per-tensor FP8 E4M3: returns (bytes uint8 like x, scale python float)."""
    lib = _lib.load()
    x = _src(x)
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    scratch = torch.empty(1, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.fa_quantize_fp8_e4m3(x.data_ptr(), _DT[x.dtype], x.numel(), 0, out.data_ptr(), scale.data_ptr(),
                                            scratch.data_ptr(), _stream(x.device)), "fa_quantize_fp8_e4m3")
    return out, scale.item()


def quantize_fp8_e4m3_per_token(x):
    """One scale per row of the last dimension (per token per head): returns (bytes uint8 like x,
    scales float32 x.shape[:-1]).  The per-tensor formula applied to each row."""
    lib = _lib.load()
    x = _src(x)
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.fa_quantize_fp8_e4m3(x.data_ptr(), _DT[x.dtype], x.numel(), x.shape[-1], out.data_ptr(),
                                            scales.data_ptr(), None, _stream(x.device)), "fa_quantize_fp8_e4m3")
    return out, scales


def dequantize_fp8_e4m3(bytes_u8, scale):
    """uint8 E4M3 bytes x scale -> float32.  `scale` is a float or a float32 tensor bytes.shape[:-1]."""
    lib = _lib.load()
    _require(bytes_u8.is_cuda and bytes_u8.dtype == torch.uint8, "bytes must be a CUDA uint8 tensor")
    b = bytes_u8.contiguous()
    out = torch.empty(b.shape, dtype=torch.float32, device=b.device)
    rows, s, per_row = None, 0.0, 0
    if isinstance(scale, torch.Tensor) and scale.numel() > 1:
        rows = scale.to(device=b.device, dtype=torch.float32).contiguous()
        per_row = b.shape[-1]
        _require(rows.numel() * per_row == b.numel(), "per-row scales must have shape bytes.shape[:-1]")
    else:
        s = float(scale)
    with torch.cuda.device(b.device):
        _lib.check(lib.fa_dequantize_fp8_e4m3(b.data_ptr(), b.numel(), s, rows.data_ptr() if rows is not None else None,
                                              per_row, out.data_ptr(), _stream(b.device)), "fa_dequantize_fp8_e4m3")
    return out


def quantize_nvfp4(x):
    """Returns (packed uint8 [..., d/2], micro uint8 [..., d/16], scale python float)."""
    lib = _lib.load()
    d = x.shape[-1]
    assert d % 16 == 0, f"head_dim {d} must be a multiple of 16 for NVFP4"
    x = _src(x)
    packed = torch.empty((*x.shape[:-1], d // 2), dtype=torch.uint8, device=x.device)
    micro = torch.empty((*x.shape[:-1], d // 16), dtype=torch.uint8, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    scratch = torch.empty(1, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.fa_quantize_nvfp4(x.data_ptr(), _DT[x.dtype], x.numel(), packed.data_ptr(), micro.data_ptr(),
                                         scale.data_ptr(), scratch.data_ptr(), _stream(x.device)), "fa_quantize_nvfp4")
    return packed, micro, scale.item()


def dequantize_nvfp4(packed_u8, micro_u8, scale):
    lib = _lib.load()
    _require(packed_u8.is_cuda and packed_u8.dtype == torch.uint8 and micro_u8.dtype == torch.uint8,
             "packed / micro must be CUDA uint8 tensors")
    p, m = packed_u8.contiguous(), micro_u8.contiguous()
    d = p.shape[-1] * 2
    _require(m.numel() * 16 == p.numel() * 2, "micro-scale tensor must hold one byte per 16 elements")
    out = torch.empty((*p.shape[:-1], d), dtype=torch.float32, device=p.device)
    with torch.cuda.device(p.device):
        _lib.check(lib.fa_dequantize_nvfp4(p.data_ptr(), m.data_ptr(), out.numel(), float(scale), out.data_ptr(),
                                           _stream(p.device)), "fa_dequantize_nvfp4")
    return out


# ---------------------------------------------------------------------------------------------- pager
def paged_scatter(x, page_size, block_table):
    """[B,H,N,dx] -> pool [B*n_logical, page_size, H, dx] under `block_table` [B, n_logical] int32."""
    lib = _lib.load()
    _require(x.is_cuda and x.dim() == 4, "x must be a CUDA tensor [B,H,N,dx]")
    x = x.contiguous()
    B, H, N, dx = x.shape
    n_logical = block_table.shape[1]
    num_blocks = B * n_logical
    pool = torch.empty((num_blocks, page_size, H, dx), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.fa_paged_scatter(x.data_ptr(), pool.data_ptr(), block_table.data_ptr(), B, H, N,
                                        dx * x.element_size(), page_size, n_logical, num_blocks, _stream(x.device)),
                   "fa_paged_scatter")
    return pool


def paged_gather(pool, block_table, page_size, n_k):
    """pool [num_blocks, page, H, dx] -> dense [B, H, n_k, dx] through the block table."""
    lib = _lib.load()
    _require(pool.is_cuda and pool.dim() == 4 and block_table.dtype == torch.int32, "bad pool / block_table")
    pool, block_table = pool.contiguous(), block_table.contiguous()
    B, n_logical = block_table.shape
    H, dx = pool.shape[2], pool.shape[3]
    out = torch.empty((B, H, int(n_k), dx), dtype=pool.dtype, device=pool.device)
    with torch.cuda.device(pool.device):
        _lib.check(lib.fa_paged_gather(pool.data_ptr(), out.data_ptr(), block_table.data_ptr(), B, H, int(n_k),
                                       dx * pool.element_size(), page_size, n_logical, pool.shape[0], _stream(pool.device)),
                   "fa_paged_gather")
    return out


def _permutation(B, n_logical, device, shuffle, seed):
    # same draw as the reference (paged.py:67-73): a generator on the input's device, seeded
    gen = None
    if seed is not None:
        gen = torch.Generator(device=device).manual_seed(seed)
    if shuffle:
        return torch.randperm(B * n_logical, device=device, generator=gen)
    return torch.arange(B * n_logical, device=device)


def build_paged_kv(k, v, page_size, *, shuffle=True, seed=None):
    """Returns (k_pool, v_pool, block_table, n_k) — reference fa_kernels/paged.py:48-91.  `k` and `v`
    may differ in their last dimension (the MLA pager pages nibbles and micro-scales in one call)."""
    B, H, N_k, _ = k.shape
    n_logical = (N_k + page_size - 1) // page_size
    perm = _permutation(B, n_logical, k.device, shuffle, seed)
    block_table = perm.reshape(B, n_logical).to(torch.int32).contiguous()
    return paged_scatter(k, page_size, block_table), paged_scatter(v, page_size, block_table), block_table, N_k


def build_paged_kv_fp8(k, v, page_size, *, shuffle=True, seed=None):
    """Returns (k_pool, v_pool, block_table, n_k, scale_k, scale_v) — reference paged.py:121-133."""
    k_q, scale_k = quantize_fp8_e4m3(k)
    v_q, scale_v = quantize_fp8_e4m3(v)
    k_pool, v_pool, block_table, n_k = build_paged_kv(k_q, v_q, page_size, shuffle=shuffle, seed=seed)
    return k_pool, v_pool, block_table, n_k, scale_k, scale_v


def build_paged_kv_fp8_per_token(k, v, page_size, *, shuffle=True, seed=None):
    """Per-token-per-head FP8: returns (k_pool, v_pool, block_table, n_k, k_scale_pool, v_scale_pool)
    with the scale pools float32 [num_blocks, page_size, H_kv] under the same block table."""
    if seed is None:
        seed = int(torch.randint(0, 2 ** 31 - 1, (1,)).item())
    k_q, ks = quantize_fp8_e4m3_per_token(k)
    v_q, vs = quantize_fp8_e4m3_per_token(v)
    k_pool, v_pool, block_table, n_k = build_paged_kv(k_q, v_q, page_size, shuffle=shuffle, seed=seed)
    ksp, vsp, _, _ = build_paged_kv(ks.unsqueeze(-1), vs.unsqueeze(-1), page_size, shuffle=shuffle, seed=seed)
    return k_pool, v_pool, block_table, n_k, ksp.squeeze(-1), vsp.squeeze(-1)


def build_paged_kv_nvfp4(k, v, page_size, *, shuffle=True, seed=None):
    """Returns (k_pack, k_micro, v_pack, v_micro, block_table, n_k, scale_k, scale_v) — paged.py:192-212."""
    if seed is None:
        seed = int(torch.randint(0, 2 ** 31 - 1, (1,)).item())
    k_pack, k_micro, scale_k = quantize_nvfp4(k)
    v_pack, v_micro, scale_v = quantize_nvfp4(v)
    kp, vp, block_table, n_k = build_paged_kv(k_pack, v_pack, page_size, shuffle=shuffle, seed=seed)
    km, vm, bt2, _ = build_paged_kv(k_micro, v_micro, page_size, shuffle=shuffle, seed=seed)
    assert torch.equal(block_table, bt2), "NVFP4 packed/micro pools must share one permutation"
    return kp, km, vp, vm, block_table, n_k, scale_k, scale_v


def build_paged_kv_mla(latent, page_size, *, shuffle=True, seed=None):
    """Returns (l_pack, l_micro, block_table, n_k, scale_l) — reference paged.py:287-309."""
    assert latent.dim() == 4 and latent.shape[1] == 1, \
        f"latent must be [B, 1, N_k, DQK] (one latent head); got {tuple(latent.shape)}"
    if seed is None:
        seed = int(torch.randint(0, 2 ** 31 - 1, (1,)).item())
    l_pack, l_micro, scale_l = quantize_nvfp4(latent)
    lp, lm, block_table, n_k = build_paged_kv(l_pack, l_micro, page_size, shuffle=shuffle, seed=seed)
    return lp, lm, block_table, n_k, scale_l


def append_paged_kv(x, pool, block_table, page_size, positions, *, scale_pool=None, micro_pool=None, tensor_scale=0.0):
    """Write T new tokens per sequence into a paged pool in place (the step before decode).

    x [B, H, T, d] float; positions int32 [B] = logical position of each sequence's first new token.
    The pool's dtype selects the conversion: float16 / bfloat16 (cast), uint8 with `scale_pool`
    (FP8 E4M3, one fp32 scale per token per head, as `quantize_fp8_e4m3_per_token`), uint8 with
    `micro_pool` and `tensor_scale` (NVFP4 relative to a fixed tensor scale, as `quantize_nvfp4`)."""
    import ctypes as C
    lib = _lib.load()
    x = _src(x)
    B, H, T, d = x.shape
    positions = positions.to(device=x.device, dtype=torch.int32).contiguous()
    _require(pool.is_cuda and pool.is_contiguous() and block_table.dtype == torch.int32, "pool must be contiguous CUDA, block_table int32")
    if pool.dtype == torch.float16:
        pd = _lib.FA_F16
    elif pool.dtype == torch.bfloat16:
        pd = FA_BF16
    elif pool.dtype == torch.uint8 and micro_pool is not None:
        pd = _lib.FA_NVFP4
    elif pool.dtype == torch.uint8:
        pd = _lib.FA_E4M3
        _require(scale_pool is not None, "FP8 pools need scale_pool")
    else:
        raise RuntimeError("pool must be float16, bfloat16 or uint8")
    lib.fa_kv_append.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p] + [C.c_int] * 8 + [C.c_float, C.c_void_p,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    with torch.cuda.device(x.device):
        _lib.check(lib.fa_kv_append(x.data_ptr(), _DT[x.dtype], positions.data_ptr(), block_table.data_ptr(), B, H, T, d,
                                    int(page_size), block_table.shape[1], pool.shape[0], pd, float(tensor_scale), pool.data_ptr(),
                                    scale_pool.data_ptr() if scale_pool is not None else None,
                                    micro_pool.data_ptr() if micro_pool is not None else None, None,
                                    _stream(x.device)), "fa_kv_append")
    return pool
