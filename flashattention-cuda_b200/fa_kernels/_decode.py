"""Torch-facing launcher of the paged GQA decode kernel (device memory, streams and caches only —
all arithmetic happens in libfa_b200.so).

Mirrors the host entry of the reference kernels (kernels/v8_gqa_ss/gqa_ss_attention.cu:264-337):
same argument checks with the same meaning, output is a fresh tensor [B, H_q, N_q, d], inputs are not
modified, work goes to torch's current stream without a host sync.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib, _status
from ._lib import FA_BF16, FA_E4M3, FA_F16, FA_F32, FA_NVFP4

_TORCH_TO_FA = {torch.float16: FA_F16, torch.bfloat16: FA_BF16, torch.float32: FA_F32}

_plan_cache: dict = {}
_workspace: dict = {}
_PLAN_CACHE_MAX = 64


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def sm_count(device) -> int:
    key = str(device)
    if key not in _sm_count:
        n = C.c_int(0)
        with torch.cuda.device(device):
            _lib.check(_lib.load().fa_device_sm_count(C.byref(n)), "fa_device_sm_count")
        _sm_count[key] = n.value
    return _sm_count[key]


def plan(seq_lens, n_k: int, B: int, H_kv: int, rows: int, page_size: int, device, chunk_hint: int = 0,
         ctas_per_sm: int = 3):
    """Return (items_device_tensor, n_items, n_slots, max_range_keys); cached per argument set.

    `seq_lens` is None (every sequence has n_k keys) or a tuple of B ints.  The planner counts three CTA
    slots per SM; a kernel that fits fewer (`ctas_per_sm`) is planned for proportionally fewer SMs.
    The device copy is uploaded on the current stream, so the cache is per stream as well: a kernel on
    another stream would have no dependency on that upload."""
    key = (seq_lens, n_k, B, H_kv, rows, page_size, str(device), torch.cuda.current_stream(device).cuda_stream,
           chunk_hint, ctas_per_sm)
    hit = _plan_cache.get(key)
    if hit is not None:
        return hit
    lib = _lib.load()
    lens_arr = None
    lens_ptr = None
    if seq_lens is not None:
        lens_arr = (C.c_int32 * B)(*seq_lens)
        lens_ptr = C.cast(lens_arr, C.c_void_p)
    cap = lib.fa_decode_plan_max_items(lens_ptr, int(n_k), B, page_size)
    host, done = _staging(device, cap)
    n_items, max_range = C.c_int(0), C.c_int(0)
    sms = sm_count(device) if int(ctas_per_sm) == 3 else -sm_count(device) * int(ctas_per_sm)
    _lib.check(lib.fa_decode_plan(lens_ptr, int(n_k), B, H_kv, rows, page_size, sms, chunk_hint,
                                  host.data_ptr(), cap, C.byref(n_items), C.byref(max_range)), "fa_decode_plan")
    n = n_items.value
    items = torch.empty((n, 8), dtype=torch.int32, device=device)
    items.copy_(host[:n], non_blocking=True)
    done.record(torch.cuda.current_stream(device))
    n_slots = n if n > B else 0
    out = (items, n, n_slots, max_range.value, None)
    if len(_plan_cache) >= _PLAN_CACHE_MAX:
        _plan_cache.pop(next(iter(_plan_cache)))
    _plan_cache[key] = out
    return out


_STAGING_SLOTS = 8
_staging_ring: dict = {}
_sm_count: dict = {}


def _staging(device, cap: int):
    """A pinned host buffer for one plan upload, from a small per-device ring.  Pinned allocations are
    slow, so buffers are reused; each slot carries the event of its last upload and is only handed out
    again after that copy has finished."""
    key = str(device)
    ring = _staging_ring.setdefault(key, {"next": 0, "slots": [None] * _STAGING_SLOTS})
    i = ring["next"]
    ring["next"] = (i + 1) % _STAGING_SLOTS
    slot = ring["slots"][i]
    if slot is None or slot[0].shape[0] < cap:
        slot = (torch.empty((max(cap, 1024), 8), dtype=torch.int32, pin_memory=True), torch.cuda.Event())
        ring["slots"][i] = slot
    else:
        slot[1].synchronize()
    return slot


def workspace(device, nbytes: int, n_counters: int):
    """(partials uint8 tensor, counters int32 tensor), one pair per (device, stream), grown
    geometrically.  The counters are allocated zeroed and the kernel hands them back zeroed; word 0 is
    the device status word (see _status.py)."""
    key = (str(device), torch.cuda.current_stream(device).cuda_stream)
    ws, cnt = _workspace.get(key, (None, None))
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(int(nbytes * 1.5), 1 << 20), dtype=torch.uint8, device=device)
    if cnt is None or cnt.numel() < n_counters:
        cnt = torch.zeros(max(int(n_counters * 2), 1 << 14), dtype=torch.int32, device=device)
        _status.register(cnt)
    _workspace[key] = (ws, cnt)
    return ws, cnt


def _lens_tuple(n_k, B):
    """n_k: int -> (None, n_k); sequence / tensor of B ints -> (tuple, max)."""
    if isinstance(n_k, torch.Tensor):
        n_k = n_k.detach().cpu().tolist()
    if isinstance(n_k, (list, tuple)):
        _require(len(n_k) == B, f"per-sequence n_k must have B={B} entries; got {len(n_k)}")
        t = tuple(int(x) for x in n_k)
        return t, (max(t) if t else 0)
    return None, int(n_k)


def paged_decode(q, k_pool, v_pool, block_table, page_size, n_k, scale, causal=False, q_offset=0, *,
                 kv_format="f16", k_micro=None, v_micro=None, scale_k=1.0, scale_v=1.0,
                 k_token_scale=None, v_token_scale=None, out_dtype=None, return_lse=False,
                 chunk_hint=0, variant=0, out=None, lse_out=None):
    lib = _lib.load()
    _require(q.is_cuda and k_pool.is_cuda and v_pool.is_cuda and block_table.is_cuda,
             "q, k_pool, v_pool, block_table must be CUDA tensors")
    _require(q.dim() == 4, "q must be [B,H_q,N_q,d]")
    _require(k_pool.dim() == 4 and v_pool.dim() == 4, "k_pool, v_pool must be [num_blocks, page_size, H_kv, d]")
    _require(block_table.dim() == 2, "block_table must be [B, n_logical]")
    _require(block_table.dtype == torch.int32, "block_table must be int32")
    page_size = int(page_size)
    B, H_q, N_q, d = q.shape
    H_kv = k_pool.shape[2]
    _require(k_pool.shape[2] == v_pool.shape[2], "k_pool/v_pool must share H_kv")
    _require(H_kv >= 1 and H_q % H_kv == 0,
             f"H_q must be a positive multiple of H_kv (GQA group factor G = H_q/H_kv); got H_q={H_q} H_kv={H_kv}")
    _require(k_pool.shape[1] == page_size and v_pool.shape[1] == page_size,
             "k_pool/v_pool page_size dim must equal page_size argument")
    _require(block_table.shape[0] == B, "block_table must have B rows")
    n_logical = block_table.shape[1]
    lens, n_max = _lens_tuple(n_k, B)
    _require(n_logical * page_size >= n_max, "block_table n_logical*page_size must cover N_k logical positions")
    _require(d in (64, 128), f"paged decode supports head_dim 64 or 128 (got {d})")

    if kv_format in ("f16", "bf16"):
        _require(k_pool.shape[3] == d and v_pool.shape[3] == d, "pool head_dim must equal q's d")
        # the reference converts q and both pools to half on every call (gqa_ss_attention.cu:293-295);
        # fp16 / bf16 pools are used as they are, anything else is converted to fp16 the same way
        if k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16:
            kv_dt, q_t = FA_BF16, torch.bfloat16
        else:
            kv_dt, q_t = FA_F16, torch.float16
            k_pool, v_pool = k_pool.to(torch.float16), v_pool.to(torch.float16)
    elif kv_format == "e4m3":
        _require(k_pool.dtype == torch.uint8 and v_pool.dtype == torch.uint8,
                 "FP8 pools must be uint8 (E4M3 bytes); build with build_paged_kv_fp8")
        _require(k_pool.shape[3] == d and v_pool.shape[3] == d, "pool head_dim must equal q's d")
        kv_dt, q_t = FA_E4M3, torch.float16
    elif kv_format == "nvfp4":
        _require(k_pool.dtype == torch.uint8 and v_pool.dtype == torch.uint8,
                 "NVFP4 pools must be uint8 (packed nibbles); build with build_paged_kv_nvfp4")
        _require(k_micro is not None and v_micro is not None and k_micro.dtype == torch.uint8
                 and v_micro.dtype == torch.uint8, "NVFP4 micro-scale pools must be uint8 (E4M3 bytes)")
        _require(k_pool.shape[3] == d // 2 and v_pool.shape[3] == d // 2,
                 "packed pool width must equal d/2 (two NVFP4 nibbles per byte)")
        _require(k_micro.shape[3] == d // 16 and v_micro.shape[3] == d // 16,
                 "micro-scale pool width must equal d/16 (one E4M3 scale per 16-element block)")
        _require(tuple(k_micro.shape[:3]) == tuple(k_pool.shape[:3]) and tuple(v_micro.shape[:3]) == tuple(v_pool.shape[:3]),
                 "packed and micro-scale pools must share [num_blocks, page_size, H_kv]")
        kv_dt, q_t = FA_NVFP4, torch.float16
        k_micro, v_micro = k_micro.contiguous(), v_micro.contiguous()
    else:
        raise RuntimeError(f"unknown kv_format {kv_format!r}")
    _require(k_pool.shape[0] == v_pool.shape[0], "k_pool/v_pool must share num_blocks")

    q = q.contiguous().to(q_t)
    k_pool, v_pool = k_pool.contiguous(), v_pool.contiguous()
    block_table = block_table.contiguous()
    dev = q.device
    if out_dtype is None:
        out_dtype = torch.float32                       # the reference returns fp32 (gqa_ss_attention.cu:296)
    _require(out_dtype in _TORCH_TO_FA, "out_dtype must be float32, float16 or bfloat16")
    if out is not None:            # caller-provided destination (e.g. a slice of a communication buffer)
        _require(out.is_cuda and out.is_contiguous() and out.numel() == B * H_q * N_q * d and out.dtype == out_dtype,
                 "out= must be a contiguous CUDA tensor of B*H_q*N_q*d elements in out_dtype")
    else:
        out = torch.empty((B, H_q, N_q, d), dtype=out_dtype, device=dev)
    if lse_out is not None:
        _require(lse_out.is_cuda and lse_out.is_contiguous() and lse_out.numel() == B * H_q * N_q
                 and lse_out.dtype == torch.float32, "lse_out= must be a contiguous CUDA float32 tensor of B*H_q*N_q")
        lse, return_lse = lse_out, True
    else:
        lse = torch.empty((B, H_q, N_q), dtype=torch.float32, device=dev) if return_lse else None

    q_offsets_t = None
    if isinstance(q_offset, torch.Tensor):
        q_offsets_t = q_offset.to(device=dev, dtype=torch.int32).contiguous()
        _require(q_offsets_t.numel() == B, "per-sequence q_offset must have B entries")
        q_offset = 0
    G = H_q // H_kv
    # the fp16 / bf16 kernel at d = 128 keeps three 32 KB stages per CTA: two CTAs per SM, the others three
    ctas = 2 if (kv_format in ("f16", "bf16") and d == 128) else 3
    # E4M3 pools on pages >= 64 with one query position run on the tcgen05 kernel: one CTA per SM
    if (kv_format == "e4m3" and d == 128 and N_q == 1 and G <= 8 and page_size >= 64
            and page_size & (page_size - 1) == 0 and int(variant) not in (2, 9)):
        ctas = 1
    items, n_items, n_slots, max_range, _ = plan(lens, n_max, B, H_kv, G * N_q, page_size, dev, int(chunk_hint), ctas)
    ws, cnt = workspace(dev, lib.fa_decode_workspace_bytes(n_slots, H_q, N_q, d),
                        lib.fa_decode_counters_len(B, H_q, H_kv, N_q))

    a = _lib.DecodeArgs()
    a.q, a.q_dtype = q.data_ptr(), _TORCH_TO_FA[q_t]
    a.k_pool, a.v_pool, a.kv_dtype = k_pool.data_ptr(), v_pool.data_ptr(), kv_dt
    a.k_micro = k_micro.data_ptr() if k_micro is not None else None
    a.v_micro = v_micro.data_ptr() if v_micro is not None else None
    a.k_scale, a.v_scale = float(scale_k), float(scale_v)
    if k_token_scale is not None:
        _require(kv_format == "e4m3" and v_token_scale is not None, "per-token scales need e4m3 pools and both K and V")
        k_token_scale = k_token_scale.contiguous().float()
        v_token_scale = v_token_scale.contiguous().float()
        _require(tuple(k_token_scale.shape) == tuple(k_pool.shape[:3]) and tuple(v_token_scale.shape) == tuple(v_pool.shape[:3]),
                 "per-token scales must be [num_blocks, page_size, H_kv]")
        a.k_token_scale, a.v_token_scale = k_token_scale.data_ptr(), v_token_scale.data_ptr()
    a.block_table, a.n_logical, a.num_blocks, a.page_size = block_table.data_ptr(), n_logical, k_pool.shape[0], page_size
    a.B, a.H_q, a.H_kv, a.N_q, a.D = B, H_q, H_kv, N_q, d
    a.softmax_scale, a.causal, a.q_offset = float(scale), int(bool(causal)), int(q_offset)
    a.q_offsets = q_offsets_t.data_ptr() if q_offsets_t is not None else None
    a.items, a.n_items, a.n_slots, a.max_range_keys = items.data_ptr(), n_items, n_slots, max_range
    a.out, a.out_dtype = out.data_ptr(), _TORCH_TO_FA[out_dtype]
    a.lse = lse.data_ptr() if lse is not None else None
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.counters, a.counters_len = cnt.data_ptr(), cnt.numel()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    a.variant = int(variant)
    with torch.cuda.device(dev):
        _lib.check(lib.fa_paged_decode_fwd(C.byref(a)), "fa_paged_decode_fwd")
    _status.after_call(dev)
    return (out, lse) if return_lse else out


def merge_partials(o_parts, lse_parts, out_dtype=torch.float32, return_lse=False):
    """o_parts [S, ..., D] fp32 normalised partial outputs, lse_parts [S, ...] -> merged [..., D].

    The parts may be strided views of one gathered buffer (dim 0 stride arbitrary, the rest dense)."""
    lib = _lib.load()
    _require(o_parts.is_cuda and lse_parts.is_cuda, "partials must be CUDA tensors")
    _require(o_parts.dtype == torch.float32 and lse_parts.dtype == torch.float32, "partials must be float32")
    S, D = o_parts.shape[0], o_parts.shape[-1]
    if not (o_parts[0].is_contiguous() and lse_parts[0].is_contiguous()):
        o_parts, lse_parts = o_parts.contiguous(), lse_parts.contiguous()
    rows = lse_parts[0].numel()
    _require(o_parts[0].numel() == rows * D and lse_parts.shape[0] == S, "o_parts / lse_parts shapes disagree")
    o_stride = o_parts.stride(0) if S > 1 else rows * D
    l_stride = lse_parts.stride(0) if S > 1 else rows
    out = torch.empty(o_parts.shape[1:], dtype=out_dtype, device=o_parts.device)
    lse = torch.empty(lse_parts.shape[1:], dtype=torch.float32, device=o_parts.device) if return_lse else None
    with torch.cuda.device(o_parts.device):
        _lib.check(lib.fa_merge_partials(o_parts.data_ptr(), lse_parts.data_ptr(), S, rows, D, o_stride, l_stride,
                                         out.data_ptr(), _TORCH_TO_FA[out_dtype], lse.data_ptr() if lse is not None else None,
                                         torch.cuda.current_stream(o_parts.device).cuda_stream), "fa_merge_partials")
    return (out, lse) if return_lse else out


class DecodeHostArgs(C.Structure):
    _fields_ = [
        ("dev", _lib.DecodeArgs),
        ("q_host", C.c_void_p), ("q_bytes", C.c_size_t),
        ("block_table_host", C.c_void_p), ("block_table_bytes", C.c_size_t),
        ("seq_lens_host", C.c_void_p), ("n_k", C.c_int),
        ("out_host", C.c_void_p), ("out_bytes", C.c_size_t),
        ("items_host", C.c_void_p), ("max_items", C.c_int), ("chunk_hint", C.c_int),
    ]


class HostDecodeStep:
    """A paged GQA decode step that starts and ends in HOST memory (C ABI `fa_paged_decode_host`): one call
    enqueues the copies of q and the block table, the plan for this step's lengths, the decode kernel and
    the copy of the output back, with no Python or allocator work between the launches.  The fp16 / bf16
    KV pools stay resident on the device; staging buffers, plan staging, workspace and counters are
    allocated once per batch shape.  An extension: the reference's `gqa_attention`
    (fa_kernels/paged.py:379-402) takes CUDA tensors and leaves the copies to the caller.

        step = HostDecodeStep(k_pool, v_pool, page_size, B, H_q, N_q, d, n_logical)
        step(q_host, block_table_host, seq_lens_host, out_host)     # pinned CPU tensors; enqueues only
        torch.cuda.current_stream().synchronize()                   # out_host is valid now
    """

    _RING = 4

    def __init__(self, k_pool, v_pool, page_size, B, H_q, N_q, d, n_logical, *, scale=None, causal=False,
                 out_dtype=torch.float16):
        lib = _lib.load()
        lib.fa_paged_decode_host.argtypes = [C.POINTER(DecodeHostArgs)]
        _require(k_pool.is_cuda and v_pool.is_cuda and k_pool.dtype == v_pool.dtype
                 and k_pool.dtype in (torch.float16, torch.bfloat16), "HostDecodeStep takes fp16 or bf16 CUDA pools")
        _require(k_pool.dim() == 4 and k_pool.shape[1] == page_size and k_pool.shape[3] == d and v_pool.shape == k_pool.shape,
                 "pools must be [num_blocks, page_size, H_kv, d]")
        _require(out_dtype in _TORCH_TO_FA, "out_dtype must be float32, float16 or bfloat16")
        dev = k_pool.device
        H_kv = k_pool.shape[2]
        _require(H_q % H_kv == 0, "H_q must be a multiple of H_kv")
        self.lib, self.dev, self.shape = lib, dev, (B, H_q, N_q, d)
        self.k_pool, self.v_pool = k_pool.contiguous(), v_pool.contiguous()
        self.q_t = k_pool.dtype
        self.out_dtype = out_dtype
        self.n_logical = int(n_logical)
        self.q_dev = torch.empty((B, H_q, N_q, d), dtype=self.q_t, device=dev)
        self.bt_dev = torch.empty((B, n_logical), dtype=torch.int32, device=dev)
        self.out_dev = torch.empty((B, H_q, N_q, d), dtype=out_dtype, device=dev)
        self.max_items = int(lib.fa_decode_plan_max_items(None, n_logical * page_size, B, page_size))
        self.items_dev = torch.empty((self.max_items, 8), dtype=torch.int32, device=dev)
        self.items_host = [torch.empty((self.max_items, 8), dtype=torch.int32).pin_memory() for _ in range(self._RING)]
        self.items_done = [None] * self._RING
        self.turn = 0
        self.ws = torch.empty(int(lib.fa_decode_workspace_bytes(self.max_items, H_q, N_q, d)), dtype=torch.uint8, device=dev)
        self.cnt = torch.zeros(int(lib.fa_decode_counters_len(B, H_q, H_kv, N_q)), dtype=torch.int32, device=dev)
        _status.register(self.cnt)
        h = DecodeHostArgs()
        a = h.dev
        a.q, a.q_dtype = self.q_dev.data_ptr(), _TORCH_TO_FA[self.q_t]
        a.k_pool, a.v_pool, a.kv_dtype = self.k_pool.data_ptr(), self.v_pool.data_ptr(), _TORCH_TO_FA[self.q_t]
        a.k_scale = a.v_scale = 1.0
        a.block_table, a.n_logical, a.num_blocks, a.page_size = self.bt_dev.data_ptr(), self.n_logical, k_pool.shape[0], int(page_size)
        a.B, a.H_q, a.H_kv, a.N_q, a.D = B, H_q, H_kv, N_q, d
        a.softmax_scale = float(scale) if scale is not None else 1.0 / d ** 0.5
        a.causal, a.q_offset = int(bool(causal)), 0
        a.items = self.items_dev.data_ptr()
        a.out, a.out_dtype = self.out_dev.data_ptr(), _TORCH_TO_FA[out_dtype]
        a.workspace, a.workspace_bytes = self.ws.data_ptr(), self.ws.numel()
        a.counters, a.counters_len = self.cnt.data_ptr(), self.cnt.numel()
        h.max_items = self.max_items
        self.h = h

    def __call__(self, q_host, block_table_host, seq_lens_host, out_host, *, q_offset=0, chunk_hint=0):
        B, H_q, N_q, d = self.shape
        _require(not q_host.is_cuda and q_host.dtype == self.q_t and q_host.is_contiguous() and tuple(q_host.shape) == self.shape,
                 "q_host must be a contiguous CPU tensor [B,H_q,N_q,d] in the pools' dtype")
        _require(block_table_host.dtype == torch.int32 and block_table_host.is_contiguous()
                 and tuple(block_table_host.shape) == (B, self.n_logical), "block_table_host must be int32 [B, n_logical] on the CPU")
        _require(out_host.dtype == self.out_dtype and out_host.is_contiguous() and tuple(out_host.shape) == self.shape,
                 "out_host must be a contiguous CPU tensor [B,H_q,N_q,d] in out_dtype")
        h = self.h
        if isinstance(seq_lens_host, torch.Tensor):
            _require(seq_lens_host.dtype == torch.int32 and seq_lens_host.numel() == B and not seq_lens_host.is_cuda,
                     "seq_lens_host must be an int32 CPU tensor of B entries")
            h.seq_lens_host, h.n_k = seq_lens_host.data_ptr(), 0
        else:
            h.seq_lens_host, h.n_k = None, int(seq_lens_host)
        i = self.turn
        self.turn = (i + 1) % self._RING
        if self.items_done[i] is not None:
            self.items_done[i].synchronize()                # the plan staging slot is free once its copy has run
        stream = torch.cuda.current_stream(self.dev)
        h.q_host, h.q_bytes = q_host.data_ptr(), q_host.numel() * q_host.element_size()
        h.block_table_host, h.block_table_bytes = block_table_host.data_ptr(), block_table_host.numel() * 4
        h.out_host, h.out_bytes = out_host.data_ptr(), out_host.numel() * out_host.element_size()
        h.items_host = self.items_host[i].data_ptr()
        h.chunk_hint = int(chunk_hint)
        h.dev.q_offset = int(q_offset)
        h.dev.stream = stream.cuda_stream
        if torch.cuda.current_device() == self.dev.index:      # the usual case: no device switch on the step's path
            _lib.check(self.lib.fa_paged_decode_host(C.byref(h)), "fa_paged_decode_host")
        else:
            with torch.cuda.device(self.dev):
                _lib.check(self.lib.fa_paged_decode_host(C.byref(h)), "fa_paged_decode_host")
        if self.items_done[i] is None:
            self.items_done[i] = torch.cuda.Event()
        self.items_done[i].record(stream)
