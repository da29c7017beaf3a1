"""fa_kernels on B200 — the public API of the reference package (fa_kernels/__init__.py:14-42)
served by hand-written sm_100a kernels behind one C-ABI library.

    from fa_kernels import gqa_attention
    out = gqa_attention(q, k_pool, v_pool, block_table, page_size, n_k)

`import fa_kernels` succeeds without CUDA; the library is loaded when a kernel is first requested
and a missing library or GPU is an error, never a fallback.
"""

from __future__ import annotations

from .config import AttnConfig
from .paged import (build_paged_kv_mla, fp8_attention, gqa_attention, mla_attention, mla_tc_attention,
                    nvfp4_attention, paged_attention)

__all__ = ["attention", "paged_attention", "gqa_attention", "fp8_attention", "nvfp4_attention",
           "mla_attention", "mla_tc_attention", "build_paged_kv_mla", "AttnConfig"]

# The reference's default is its teaching baseline "v1_naive" (fa_kernels/__init__.py:23); every dense
# backend name maps to the one tensor-core kernel here.
_DEFAULT_BACKEND = "v1_naive"


def attention(q, k, v, *, causal: bool = False, scale: float | None = None, backend: str = _DEFAULT_BACKEND, **kw):
    """Scaled dot-product attention, q/k/v [B, H, N, d] CUDA tensors (reference
    fa_kernels/__init__.py:26-42).  `causal` masks key j for query i when j > i; `scale` None means
    1/sqrt(d).  Extra keywords: `out_dtype` (default float32), `return_lse`."""
    from .dispatch import get_backend

    if scale is None:
        scale = 1.0 / (q.shape[-1] ** 0.5)
    module = get_backend(backend)
    return module.forward(q, k, v, scale, causal, **kw)


def __getattr__(name):
    # extensions that need torch and the CUDA library are resolved on first use, so that
    # `import fa_kernels` keeps working without either
    if name == "HostDecodeStep":
        from ._decode import HostDecodeStep
        return HostDecodeStep
    if name in ("check_status", "read_status", "set_status_checks"):
        from . import _status
        return getattr(_status, name)
    raise AttributeError(f"module 'fa_kernels' has no attribute {name!r}")
