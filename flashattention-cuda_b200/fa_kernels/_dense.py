"""Torch-facing launcher of the dense attention kernel (csrc/prefill.cu) — the host side of the
reference's dense `forward(q, k, v, scale, causal)` (kernels/v5_wmma/wmma_attention.cu:229-263): inputs
of any float dtype are converted to half precision, the output is a fresh [B,H,N_q,d] tensor (fp32 by
default), work goes to torch's current stream."""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib, _status
from ._lib import FA_BF16, FA_F16, FA_F32

_TORCH_TO_FA = {torch.float16: FA_F16, torch.bfloat16: FA_BF16, torch.float32: FA_F32}
_words: dict = {}


class DenseArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("dtype", C.c_int),
                ("B", C.c_int), ("H", C.c_int), ("N_q", C.c_int), ("N_k", C.c_int), ("D", C.c_int),
                ("softmax_scale", C.c_float), ("causal", C.c_int),
                ("out", C.c_void_p), ("out_dtype", C.c_int), ("lse", C.c_void_p), ("status", C.c_void_p),
                ("stream", C.c_void_p)]


def status_word(device) -> torch.Tensor:
    """Device int that a kernel sets when one of its bounded pipeline waits gave up (0 = healthy)."""
    key = str(device)
    if key not in _words:
        _words[key] = torch.zeros(1, dtype=torch.int32, device=device)
        _status.register(_words[key])
    return _words[key]


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def dense_attention(q, k, v, scale, causal, *, out_dtype=None, return_lse=False):
    lib = _lib.load()
    _require(q.is_cuda and k.is_cuda and v.is_cuda, "q, k, v must be CUDA tensors")
    _require(q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q, k, v must be [B,H,N,d]")
    B, H, N_q, d = q.shape
    _require(tuple(k.shape) == tuple(v.shape) and k.shape[0] == B and k.shape[1] == H and k.shape[3] == d,
             "k, v must be [B,H,N_k,d] matching q's B, H, d")
    N_k = k.shape[2]
    _require(d in (64, 128), f"dense attention supports head_dim 64 or 128 (got {d})")
    t = torch.bfloat16 if (q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16) \
        else torch.float16
    q, k, v = (x.contiguous().to(t) for x in (q, k, v))
    if out_dtype is None:
        out_dtype = torch.float32
    _require(out_dtype in _TORCH_TO_FA, "out_dtype must be float32, float16 or bfloat16")
    dev = q.device
    out = torch.empty((B, H, N_q, d), dtype=out_dtype, device=dev)
    lse = torch.empty((B, H, N_q), dtype=torch.float32, device=dev) if return_lse else None
    a = DenseArgs()
    a.q, a.k, a.v, a.dtype = q.data_ptr(), k.data_ptr(), v.data_ptr(), _TORCH_TO_FA[t]
    a.B, a.H, a.N_q, a.N_k, a.D = B, H, N_q, N_k, d
    a.softmax_scale, a.causal = float(scale), int(bool(causal))
    a.out, a.out_dtype = out.data_ptr(), _TORCH_TO_FA[out_dtype]
    a.lse = lse.data_ptr() if lse is not None else None
    a.status = status_word(dev).data_ptr()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        _lib.check(lib.fa_dense_fwd(C.byref(a)), "fa_dense_fwd")
    _status.after_call(dev)
    return (out, lse) if return_lse else out
