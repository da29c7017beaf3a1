"""fa_kernels on B200 — the public API of the reference package (fa_kernels/__init__.py:14-42)
served by hand-written sm_100a kernels behind one C-ABI library.

    from fa_kernels import gqa_attention
    out = gqa_attention(q, k_pool, v_pool, block_table, page_size, n_k)

`import fa_kernels` succeeds without CUDA; the library is loaded when a kernel is first requested
and a missing library or GPU is an error, never a fallback.
"""

from __future__ import annotations

from .config import AttnConfig
from .paged import fp8_attention, gqa_attention, nvfp4_attention, paged_attention

__all__ = ["paged_attention", "gqa_attention", "fp8_attention", "nvfp4_attention", "AttnConfig"]
