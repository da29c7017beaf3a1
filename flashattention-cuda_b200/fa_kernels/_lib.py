"""ctypes binding of libfa_b200.so — the prebuilt C-ABI library that stands where the reference
JIT-loads one pybind module per kernel (bindings/load.py:107-131).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

FA_F16, FA_BF16, FA_F32, FA_E4M3, FA_NVFP4 = 0, 1, 2, 3, 4

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_DEFAULT_LIB = os.path.join(_PKG_DIR, "libfa_b200.so")

_lock = threading.Lock()
_lib = None


class DecodeItem(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("b", "k_begin", "k_end", "slot_base", "n_split", "split", "pad0", "pad1")]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_dtype", C.c_int),
        ("k_pool", C.c_void_p), ("v_pool", C.c_void_p), ("kv_dtype", C.c_int),
        ("k_micro", C.c_void_p), ("v_micro", C.c_void_p),
        ("k_scale", C.c_float), ("v_scale", C.c_float),
        ("k_token_scale", C.c_void_p), ("v_token_scale", C.c_void_p),
        ("block_table", C.c_void_p), ("n_logical", C.c_int), ("num_blocks", C.c_int),
        ("page_size", C.c_int),
        ("B", C.c_int), ("H_q", C.c_int), ("H_kv", C.c_int), ("N_q", C.c_int), ("D", C.c_int),
        ("softmax_scale", C.c_float), ("causal", C.c_int), ("q_offset", C.c_int),
        ("q_offsets", C.c_void_p),
        ("items", C.c_void_p), ("n_items", C.c_int), ("n_slots", C.c_int), ("max_range_keys", C.c_int),
        ("out", C.c_void_p), ("out_dtype", C.c_int), ("lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("counters", C.c_void_p), ("counters_len", C.c_size_t),
        ("stream", C.c_void_p), ("variant", C.c_int),
    ]


def lib_path() -> str:
    return os.environ.get("FA_B200_LIB", _DEFAULT_LIB)


def _declare(lib):
    lib.fa_last_error.restype = C.c_char_p
    lib.fa_last_error.argtypes = []
    lib.fa_version.restype = C.c_int
    lib.fa_status_text.restype = C.c_char_p
    lib.fa_status_text.argtypes = [C.c_int]
    lib.fa_device_sm_count.argtypes = [C.POINTER(C.c_int)]
    lib.fa_decode_plan.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    lib.fa_decode_plan_max_items.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
    lib.fa_decode_workspace_bytes.restype = C.c_size_t
    lib.fa_decode_workspace_bytes.argtypes = [C.c_int] * 4
    lib.fa_decode_counters_len.restype = C.c_size_t
    lib.fa_decode_counters_len.argtypes = [C.c_int] * 4
    lib.fa_paged_decode_fwd.argtypes = [C.POINTER(DecodeArgs)]
    lib.fa_merge_partials.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int64, C.c_int64,
                                      C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    for name, argtypes in _OPTIONAL.items():
        if hasattr(lib, name):
            getattr(lib, name).argtypes = argtypes


# entry points declared by later sections of include/fa_b200.h (argtypes filled in when present)
_OPTIONAL: dict = {
    "fa_mla_decode_fwd": [C.c_void_p],
    "fa_dense_fwd": [C.c_void_p],
    "fa_paged_decode_fwd_static": [C.POINTER(DecodeArgs)],
    "fa_paged_decode_static_status": [C.POINTER(C.c_int32), C.c_int, C.c_void_p],
    "fa_selftest_bounded_wait": [C.c_void_p, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p],
    "fa_quantize_fp8_e4m3": [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p],
    "fa_dequantize_fp8_e4m3": [C.c_void_p, C.c_int64, C.c_float, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p],
    "fa_quantize_nvfp4": [C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p],
    "fa_dequantize_nvfp4": [C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_void_p, C.c_void_p],
    "fa_paged_scatter": [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 7 + [C.c_void_p],
    "fa_paged_gather": [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 7 + [C.c_void_p],
}


def load():
    """Load (once) and return the ctypes handle.  Raises RuntimeError when the library is absent —
    the package has no other execution path."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = lib_path()
            if not os.path.exists(path):
                raise RuntimeError(
                    f"libfa_b200.so not found at {path}; build it with "
                    f"`python flashattention-cuda_b200/build.py` (needs nvcc) or set FA_B200_LIB")
            lib = C.CDLL(path)
            _declare(lib)
            _lib = lib
    return _lib


def check(status: int, what: str = "") -> None:
    if status != 0:
        msg = load().fa_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what}: {msg}" if what else msg)
