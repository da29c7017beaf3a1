"""Paged-KV attention entry points — the import surface of the reference's fa_kernels/paged.py
(same names, argument order and meaning), running on the B200 kernels of libfa_b200.so.

Shapes (fa_kernels/paged.py:12-24 of the reference):
    q           : [B, H_q, N_q, d]                     CUDA tensor (decode: N_q = 1)
    k_pool      : [num_blocks, page_size, H_kv, d]     physical KV pool
    v_pool      : [num_blocks, page_size, H_kv, d]
    block_table : [B, n_logical] int32                 block_table[b][lb] -> physical block
    n_k         : logical KV length attended this step; an int (the reference contract) or one
                  length per sequence (list / tensor of B ints)

Keyword-only additions to every attention call: `out_dtype` (default float32 as in the reference),
`return_lse` (also return the log-sum-exp [B, H_q, N_q]).
"""

from __future__ import annotations

DEFAULT_PAGED_BACKEND = "v7_paged"
DEFAULT_GQA_BACKEND = "v8_gqa"
DEFAULT_FP8_BACKEND = "v9_fp8"
DEFAULT_NVFP4_BACKEND = "v10_nvfp4"
DEFAULT_MLA_BACKEND = "v11_mla"
DEFAULT_MLA_TC_BACKEND = "v12_mla_tc"

_E4M3_MAX = 448.0
_NVFP4_BLOCK = 16
_E2M1_MAX = 6.0
_E2M1_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def _default_scale(q, scale):
    return 1.0 / (q.shape[-1] ** 0.5) if scale is None else scale


def paged_attention(q, k_pool, v_pool, block_table, page_size, n_k, *, scale=None, causal=False,
                    q_offset=0, backend=DEFAULT_PAGED_BACKEND, **kw):
    """Paged-KV attention (reference fa_kernels/paged.py:215-234).  `causal` masks key j when
    j > query_i + q_offset; at decode set q_offset = n_k - N_q."""
    from .dispatch import get_backend
    module = get_backend(backend)
    return module.forward(q, k_pool, v_pool, block_table, int(page_size), n_k,
                          _default_scale(q, scale), causal, q_offset, **kw)


def gqa_attention(q, k_pool, v_pool, block_table, page_size, n_k, *, scale=None, causal=False,
                  q_offset=0, backend=DEFAULT_GQA_BACKEND, **kw):
    """GQA M-packed paged decode (reference fa_kernels/paged.py:379-402): the pool has H_kv heads, q has
    H_q = G * H_kv; KV head h serves query heads [h*G, h*G + G)."""
    from .dispatch import get_backend
    module = get_backend(backend)
    return module.forward(q, k_pool, v_pool, block_table, int(page_size), n_k,
                          _default_scale(q, scale), causal, q_offset, **kw)


def fp8_attention(q, k_pool, v_pool, block_table, page_size, n_k, scale_k, scale_v, *, scale=None,
                  causal=False, q_offset=0, backend=DEFAULT_FP8_BACKEND, **kw):
    """FP8 E4M3 KV-cache GQA decode (reference fa_kernels/paged.py:237-260).  Pools are uint8 E4M3
    bytes; `scale_k` / `scale_v` are the per-tensor dequant scales, or float32 tensors
    [num_blocks, page_size, H_kv] holding one scale per token per head."""
    from .dispatch import get_backend
    module = get_backend(backend)
    return module.forward(q, k_pool, v_pool, block_table, int(page_size), n_k, scale_k, scale_v,
                          _default_scale(q, scale), causal, q_offset, **kw)


def nvfp4_attention(q, k_pack, k_micro, v_pack, v_micro, block_table, page_size, n_k, scale_k, scale_v, *,
                    scale=None, causal=False, q_offset=0, backend=DEFAULT_NVFP4_BACKEND, **kw):
    """NVFP4 KV-cache GQA decode (reference fa_kernels/paged.py:263-284): packed E2M1 nibbles
    [.., d/2] + E4M3 micro-scales [.., d/16] + one fp32 scale per tensor."""
    from .dispatch import get_backend
    module = get_backend(backend)
    return module.forward(q, k_pack, k_micro, v_pack, v_micro, block_table, int(page_size), n_k,
                          float(scale_k), float(scale_v), _default_scale(q, scale), causal, q_offset, **kw)


def mla_attention(q, l_pack, l_micro, block_table, page_size, n_k, kv_lora_rank, scale_l, *, scale=None,
                  causal=False, q_offset=0, backend=DEFAULT_MLA_BACKEND, **kw):
    """MLA latent-KV decode (reference fa_kernels/paged.py:312-340): all H_q heads attend one shared
    latent; scores over DQK, output = p-weighted sum of the first `kv_lora_rank` latent dims,
    [B, H_q, N_q, kv_lora_rank].  Default scale 1/sqrt(DQK).  `l_pack` is the packed NVFP4 pool of
    `build_paged_kv_mla` with `l_micro` its micro-scales, or a bf16 / FP8 E4M3 latent pool
    [num_blocks, page_size, 1, DQK] (then `l_micro` is ignored and `scale_l` is a float or, for FP8,
    per-token float32 scales [num_blocks, page_size, 1])."""
    from .dispatch import get_backend
    module = get_backend(backend)
    return module.forward(q, l_pack, l_micro, block_table, int(page_size), n_k, int(kv_lora_rank), scale_l,
                          _default_scale(q, scale), causal, q_offset, **kw)


_MLA_TC_ENGINES = {"fp8": 0, "nvfp4": 1}


def mla_tc_attention(q, l_pack, l_micro, block_table, page_size, n_k, kv_lora_rank, scale_l, *, engine="fp8",
                     scale=None, causal=False, q_offset=0, backend=DEFAULT_MLA_TC_BACKEND, **kw):
    """Tensor-core MLA decode (reference fa_kernels/paged.py:346-376): same inputs and output as
    `mla_attention`; `engine` in {"fp8", "nvfp4"} is validated as in the reference."""
    from .dispatch import get_backend
    if engine not in _MLA_TC_ENGINES:
        raise ValueError(f"engine must be one of {sorted(_MLA_TC_ENGINES)}; got {engine!r}")
    module = get_backend(backend)
    return module.forward(q, l_pack, l_micro, block_table, int(page_size), n_k, int(kv_lora_rank), scale_l,
                          _default_scale(q, scale), causal, q_offset, int(_MLA_TC_ENGINES[engine]), **kw)


# ---- layout builders and quantisers (reference fa_kernels/paged.py:48-212, 287-309) ------------------
# Thin lazy forwards so that `import fa_kernels` needs neither torch nor the CUDA library.
def _fwd(name):
    def call(*args, **kwargs):
        from . import _formats
        return getattr(_formats, name)(*args, **kwargs)
    call.__name__ = name
    call.__doc__ = f"See fa_kernels._formats.{name} (GPU implementation of the reference helper of the same name)."
    return call


build_paged_kv = _fwd("build_paged_kv")
build_paged_kv_fp8 = _fwd("build_paged_kv_fp8")
build_paged_kv_fp8_per_token = _fwd("build_paged_kv_fp8_per_token")
build_paged_kv_nvfp4 = _fwd("build_paged_kv_nvfp4")
build_paged_kv_mla = _fwd("build_paged_kv_mla")
quantize_fp8_e4m3 = _fwd("quantize_fp8_e4m3")
quantize_fp8_e4m3_per_token = _fwd("quantize_fp8_e4m3_per_token")
dequantize_fp8_e4m3 = _fwd("dequantize_fp8_e4m3")
quantize_nvfp4 = _fwd("quantize_nvfp4")
dequantize_nvfp4 = _fwd("dequantize_nvfp4")
paged_gather = _fwd("paged_gather")
append_paged_kv = _fwd("append_paged_kv")
