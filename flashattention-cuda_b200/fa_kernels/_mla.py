"""Torch-facing launcher of the MLA latent decode kernel (csrc/mla.cu) — the host side of the
reference's `mla_attention_forward` (kernels/v11_mla/mla_attention.cu:320-409): same checks, output
O_latent [B, H_q, N_q, kv_lora_rank] (fp32 by default) on torch's current stream.

The reference stores the latent only as NVFP4 (packed nibbles + micro-scales); bf16 and FP8 E4M3
latents are accepted behind the same call, selected by the pool's dtype."""

from __future__ import annotations

import ctypes as C

import torch

from . import _decode, _lib, _status
from ._lib import FA_BF16, FA_E4M3, FA_F16, FA_F32, FA_NVFP4

_TORCH_TO_FA = {torch.float16: FA_F16, torch.bfloat16: FA_BF16, torch.float32: FA_F32}
_require = _decode._require


class MlaArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_dtype", C.c_int), ("l_pool", C.c_void_p), ("latent_dtype", C.c_int),
        ("l_micro", C.c_void_p), ("l_scale", C.c_float), ("l_token_scale", C.c_void_p),
        ("block_table", C.c_void_p), ("n_logical", C.c_int), ("num_blocks", C.c_int), ("page_size", C.c_int),
        ("B", C.c_int), ("H_q", C.c_int), ("N_q", C.c_int), ("DQK", C.c_int), ("DV", C.c_int),
        ("softmax_scale", C.c_float), ("causal", C.c_int), ("q_offset", C.c_int), ("q_offsets", C.c_void_p),
        ("items", C.c_void_p), ("n_items", C.c_int), ("n_slots", C.c_int), ("max_range_keys", C.c_int),
        ("out", C.c_void_p), ("out_dtype", C.c_int), ("lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("counters", C.c_void_p), ("counters_len", C.c_size_t), ("stream", C.c_void_p), ("engine_hint", C.c_int),
    ]


def _expand_budget_bytes():
    """Largest bf16 copy of a quantised latent pool the tensor-core route may allocate
    (FA_B200_MLA_EXPAND_MAX_GB, default 16; 0 keeps quantised latents on the fused kernel)."""
    import os
    return int(float(os.environ.get("FA_B200_MLA_EXPAND_MAX_GB", "16")) * (1 << 30))


def mla_decode(q, l_pool, l_micro, block_table, page_size, n_k, kv_lora_rank, scale_l, scale, causal=False,
               q_offset=0, *, out_dtype=None, return_lse=False, chunk_hint=0, out=None, lse_out=None, engine_hint=0):
    lib = _lib.load()
    lib.fa_mla_counters_len.restype = C.c_size_t
    lib.fa_mla_counters_len.argtypes = [C.c_int] * 3
    lib.fa_mla_decode_fwd.argtypes = [C.POINTER(MlaArgs)]
    lib.fa_mla_workspace_bytes.restype = C.c_size_t
    lib.fa_mla_workspace_bytes.argtypes = [C.c_int] * 4
    _require(q.is_cuda and l_pool.is_cuda and block_table.is_cuda, "q, l_pool, l_scale, block_table must be CUDA tensors")
    _require(q.dim() == 4, "q (q_absorbed) must be [B,H_q,N_q,DQK]")
    _require(l_pool.dim() == 4, "l_pool must be [num_blocks, page_size, H_kv=1, *]")
    _require(block_table.dim() == 2 and block_table.dtype == torch.int32, "block_table must be int32 [B, n_logical]")
    page_size = int(page_size)
    B, H_q, N_q, DQK = q.shape
    DV = int(kv_lora_rank)
    _require(l_pool.shape[2] == 1, f"MLA latent pool must have exactly one (latent) head; got H_kv={l_pool.shape[2]}")
    _require(DQK % 16 == 0, f"DQK (latent width) must be a multiple of the NVFP4 block (16); got {DQK}")
    _require(1 <= DV <= DQK and DV % 32 == 0, f"kv_lora_rank (DV) must be in [1,DQK], a multiple of 32; got {DV} DQK={DQK}")
    _require(l_pool.shape[1] == page_size, "latent pools must share [num_blocks, page_size, 1, *]")
    _require(block_table.shape[0] == B, "block_table must have B rows")
    n_logical = block_table.shape[1]
    lens, n_max = _decode._lens_tuple(n_k, B)
    _require(n_logical * page_size >= n_max, "block_table n_logical*page_size must cover N_k logical positions")

    tok_scale = None
    l_scale = 1.0
    if l_pool.dtype == torch.bfloat16:
        _require(l_pool.shape[3] == DQK, "bf16 latent pool width must equal DQK")
        fmt, q_t = FA_BF16, torch.bfloat16
        l_micro = None
        l_scale = float(scale_l) if not isinstance(scale_l, torch.Tensor) else 1.0
    elif l_pool.dtype == torch.uint8 and l_pool.shape[3] == DQK:
        fmt, q_t = FA_E4M3, torch.float16
        l_micro = None
        if isinstance(scale_l, torch.Tensor) and scale_l.numel() > 1:
            tok_scale = scale_l.to(device=q.device, dtype=torch.float32).contiguous()
            _require(tok_scale.numel() == l_pool.shape[0] * page_size, "per-token latent scales must be [num_blocks, page_size, 1]")
        else:
            l_scale = float(scale_l)
    elif l_pool.dtype == torch.uint8:
        _require(l_pool.shape[3] == DQK // 2, "packed latent pool width must equal DQK/2 (two NVFP4 nibbles per byte)")
        _require(l_micro is not None and l_micro.dtype == torch.uint8, "l_scale must be uint8 (E4M3 micro-scale bytes)")
        _require(l_micro.dim() == 4 and l_micro.shape[3] == DQK // 16 and l_micro.shape[1] == page_size and l_micro.shape[2] == 1,
                 "micro-scale pool width must equal DQK/16 (one E4M3 scale per 16-element block)")
        fmt, q_t = FA_NVFP4, torch.float16
        l_micro = l_micro.contiguous()
        l_scale = float(scale_l)
    else:
        raise RuntimeError("l_pool must be bfloat16, uint8 E4M3 [.., DQK] or uint8 packed NVFP4 [.., DQK/2]")

    q_in = q
    q = q.contiguous().to(q_t)
    l_pool, block_table = l_pool.contiguous(), block_table.contiguous()
    dev = q.device
    if out_dtype is None:
        out_dtype = torch.float32
    _require(out_dtype in _TORCH_TO_FA, "out_dtype must be float32, float16 or bfloat16")
    if out is None:
        out = torch.empty((B, H_q, N_q, DV), dtype=out_dtype, device=dev)
    else:
        _require(out.is_cuda and out.is_contiguous() and out.numel() == B * H_q * N_q * DV and out.dtype == out_dtype,
                 "out= must be a contiguous CUDA tensor of B*H_q*N_q*DV elements in out_dtype")
    if lse_out is not None:
        _require(lse_out.is_contiguous() and lse_out.numel() == B * H_q * N_q and lse_out.dtype == torch.float32,
                 "lse_out= must be a contiguous float32 tensor of B*H_q*N_q")
        lse, return_lse = lse_out, True
    else:
        lse = torch.empty((B, H_q, N_q), dtype=torch.float32, device=dev) if return_lse else None
    q_offsets_t = None
    if isinstance(q_offset, torch.Tensor):
        q_offsets_t = q_offset.to(device=dev, dtype=torch.int32).contiguous()
        q_offset = 0

    rows32 = 16 * ((H_q * N_q + 31) // 32)          # the planner counts 16-row tiles; this kernel uses 32
    tc_geometry = (DQK == 576 and DV == 512 and page_size % 64 == 0 and page_size & (page_size - 1) == 0
                   and engine_hint != 2)
    # An FP8 latent of that geometry with enough head rows to fill an MMA tile runs on the tensor-core kernel
    # as it is (tcgen05 kind::f8f6f4 on the stored bytes, csrc/mla_pair_f8.cu).  An NVFP4 latent reaches the
    # tensor-core kernel through a transient bf16 copy of the tokens in use (one elementwise pass,
    # fa_mla_expand_latent) when the copy fits the budget.  Everything else runs on the fused mma.sync kernel,
    # which dequantises tile by tile.
    fused_fp8 = tc_geometry and fmt == FA_E4M3 and H_q * N_q >= 64 and l_pool.data_ptr() % 16 == 0
    expand = (tc_geometry and fmt == FA_NVFP4 and H_q * N_q >= 64
              and l_pool.shape[0] * page_size * DQK * 2 <= _expand_budget_bytes())
    tc_shape = tc_geometry and (fmt == FA_BF16 or expand or fused_fp8)
    if tc_shape:
        # the tensor-core kernel stages a bounded number of block-table entries per CTA pair: bound the ranges
        cap = lib.fa_mla_pair_max_range(page_size)
        if chunk_hint:
            chunk_hint = min(int(chunk_hint), cap)
        else:
            # A key range costs tens of microseconds of pipeline fill, drain and merge in this kernel (measured),
            # so sequences stay whole while there is one (sequence, 128-row tile) unit per CTA pair.  With fewer
            # units -- what one GPU of several sees of a sharded batch -- the sequences are cut into equal
            # ranges under the shortest common cap that fills one wave of pairs, or two waves when more than
            # half of the pairs would hold a whole sequence anyway (measured on 16 / 32 / 64 sequences of
            # 4096-32768 keys: 139 / 232 / 397 us against 197 / 277 / 434 us for two ranges per pair).
            slots = max(1, _decode.sm_count(dev) // 2)
            tiles = (H_q * N_q + 127) // 128
            units = B * tiles
            if units >= slots:
                chunk_hint = cap
            else:
                seq = lens if lens is not None else (n_max,) * B
                budget = slots if 2 * units <= slots else 2 * slots
                lo, hi = 8, max(8, cap // 128)                   # cap in 128-key tiles; at least 1024 keys
                while lo < hi:
                    mid = (lo + hi) // 2
                    if sum(max(1, -(-n // (mid * 128))) for n in seq) * tiles <= budget:
                        hi = mid
                    else:
                        lo = mid + 1
                chunk_hint = min(cap, lo * 128)
    items, n_items, n_slots, max_range, _ = _decode.plan(lens, n_max, B, 1, rows32, page_size, dev, int(chunk_hint))
    ws, cnt = _decode.workspace(dev, lib.fa_mla_workspace_bytes(n_slots, H_q, N_q, DV),
                                lib.fa_mla_counters_len(B, H_q, N_q))
    if expand:
        lib.fa_mla_expand_latent.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_int, C.c_int,
                                             C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        wide = torch.empty((l_pool.shape[0], page_size, 1, DQK), dtype=torch.bfloat16, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.fa_mla_expand_latent(l_pool.data_ptr(), fmt, l_micro.data_ptr() if l_micro is not None else None,
                                                tok_scale.data_ptr() if tok_scale is not None else None, float(l_scale),
                                                block_table.data_ptr(), n_logical, l_pool.shape[0], page_size, items.data_ptr(),
                                                n_items, DQK, wide.data_ptr(), torch.cuda.current_stream(dev).cuda_stream),
                       "fa_mla_expand_latent")
        l_pool, l_micro, tok_scale, l_scale, fmt, q_t = wide, None, None, 1.0, FA_BF16, torch.bfloat16
        q = q_in.contiguous().to(torch.bfloat16)
    a = MlaArgs()
    a.q, a.q_dtype = q.data_ptr(), _TORCH_TO_FA[q_t]
    a.l_pool, a.latent_dtype = l_pool.data_ptr(), fmt
    a.l_micro = l_micro.data_ptr() if l_micro is not None else None
    a.l_scale = l_scale
    a.l_token_scale = tok_scale.data_ptr() if tok_scale is not None else None
    a.block_table, a.n_logical, a.num_blocks, a.page_size = block_table.data_ptr(), n_logical, l_pool.shape[0], page_size
    a.B, a.H_q, a.N_q, a.DQK, a.DV = B, H_q, N_q, DQK, DV
    a.softmax_scale, a.causal, a.q_offset = float(scale), int(bool(causal)), int(q_offset)
    a.q_offsets = q_offsets_t.data_ptr() if q_offsets_t is not None else None
    a.items, a.n_items, a.n_slots, a.max_range_keys = items.data_ptr(), n_items, n_slots, max_range
    a.out, a.out_dtype = out.data_ptr(), _TORCH_TO_FA[out_dtype]
    a.lse = lse.data_ptr() if lse is not None else None
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.counters, a.counters_len = cnt.data_ptr(), cnt.numel()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    a.engine_hint = int(engine_hint)
    with torch.cuda.device(dev):
        _lib.check(lib.fa_mla_decode_fwd(C.byref(a)), "fa_mla_decode_fwd")
    _status.after_call(dev)
    return (out, lse) if return_lse else out
