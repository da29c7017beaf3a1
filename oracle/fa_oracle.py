"""CPU oracle for the fa_kernels attention path (TEST INFRASTRUCTURE, not a product code path).

A numpy restatement of the reference project's CPU-capable correctness anchors and data-format
helpers.  Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import
this module; the product package never does (it fails loudly when its CUDA library is missing).

Every function cites the reference file:line it follows.  Parity is PINNED: the golden fixtures
under ``tests/golden/`` were produced by importing the reference's own ``fa_kernels`` package
(see ``tests/golden/make_golden.py``) and ``tests/test_oracle_golden.py`` checks this module
against them bit-for-bit (integer/byte work) or to 1e-5 (float attention outputs).

Conventions follow the reference: tensors are ``[B, H, N, d]`` row-major; pools are
``[num_blocks, page_size, H_kv, dx]``; ``block_table`` is int32 ``[B, n_logical]``.
"""

from __future__ import annotations

import numpy as np

# fa_kernels/paged.py:34-45 — format constants.
E4M3_MAX = 448.0
NVFP4_BLOCK = 16
E2M1_MAX = 6.0
E2M1_LEVELS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_MIDPOINTS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)


# ----------------------------------------------------------------------------------------------
# FP8 E4M3 ("e4m3fn": no inf, 0x7F/0xFF = NaN, max normal 448) byte codec.
# The reference stores `(x / scale).to(torch.float8_e4m3fn)` (fa_kernels/paged.py:108), i.e. torch's
# float32 -> e4m3fn cast: round-to-nearest-even, NOT saturating (|x| > 464 becomes NaN).
# ----------------------------------------------------------------------------------------------
def e4m3_encode(x) -> np.ndarray:
    """float32 array -> uint8 E4M3 bytes, round-to-nearest-even, non-saturating."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    ax = np.abs(x).astype(np.float64)
    nan = np.isnan(ax)
    ax = np.where(nan, 0.0, ax)
    # exponent of the binade, clamped to the subnormal binade (2^-6): quantum is 2^(e-3)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(ax > 0, ax, 1.0)))
    e = np.maximum(e, -6.0)
    quantum = np.exp2(e - 3.0)
    val = np.rint(ax / quantum) * quantum          # np.rint is round-half-to-even
    over = val > 448.0
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(val > 0, val, 1.0)))
    e2 = np.maximum(e2, -6.0)
    is_sub = val < 2.0 ** -6
    mant_norm = np.rint((val / np.exp2(e2) - 1.0) * 8.0)
    mant_sub = np.rint(val / 2.0 ** -9)
    exp_field = np.where(is_sub, 0.0, e2 + 7.0)
    mant = np.where(is_sub, mant_sub, mant_norm)
    code = (exp_field.astype(np.int64) << 3) | mant.astype(np.int64)
    code = np.where(over | nan, 0x7F, code).astype(np.uint8)
    return (code | sign).astype(np.uint8)


def e4m3_decode(b) -> np.ndarray:
    """uint8 E4M3 bytes -> float32 (the `.view(torch.float8_e4m3fn).float()` of paged.py:118)."""
    b = np.asarray(b, dtype=np.uint8)
    s = np.where(b & 0x80, -1.0, 1.0)
    e = ((b >> 3) & 0xF).astype(np.int32)
    m = (b & 0x7).astype(np.float64)
    sub = (m / 8.0) * 2.0 ** -6
    nor = (1.0 + m / 8.0) * np.exp2(e.astype(np.float64) - 7.0)
    v = np.where(e == 0, sub, nor)
    v = np.where((b & 0x7F) == 0x7F, np.nan, v)
    return (s * v).astype(np.float32)


def quantize_fp8_e4m3(x):
    """Per-tensor FP8 quantise — fa_kernels/paged.py:94-109.

    scale = float32(amax.clamp_min(1e-12) / 448) read back as a python float; the bytes are the
    e4m3 cast of the float32 quotient x / scale.
    """
    x = np.asarray(x, dtype=np.float32)
    amax = np.maximum(np.abs(x).max(), np.float32(1e-12)).astype(np.float32)
    scale = float(np.float32(amax / np.float32(E4M3_MAX)))
    q = (x / np.float32(scale)).astype(np.float32)
    return e4m3_encode(q), scale


def dequantize_fp8_e4m3(bytes_u8, scale):
    """fa_kernels/paged.py:112-118."""
    return e4m3_decode(bytes_u8) * np.float32(scale)


def quantize_fp8_e4m3_per_token(x):
    """Per-(token, head) FP8 quantise: the formula of paged.py:106-108 with amax over the last
    (head-dim) axis only.  Returns (bytes[..., d] uint8, scales[...] float32).  This granularity is
    not in the reference API; it is the long-context FP8 layout (one fp32 scale per token per head).
    """
    x = np.asarray(x, dtype=np.float32)
    amax = np.maximum(np.abs(x).max(axis=-1, keepdims=True), np.float32(1e-12)).astype(np.float32)
    scale = (amax / np.float32(E4M3_MAX)).astype(np.float32)
    q = (x / scale).astype(np.float32)
    return e4m3_encode(q), scale[..., 0]


def quantize_nvfp4(x):
    """Two-level NVFP4 quantise — fa_kernels/paged.py:136-170.

    Returns (packed[..., d/2] uint8, micro[..., d/16] uint8, scale float).  Semantics that must be
    reproduced: E2M1 rounding is a left-bisect over the midpoints (ties go to the LOWER magnitude,
    NaN sorts last -> index 7); sign bit is (y < 0); low nibble is the even element.
    """
    x = np.asarray(x, dtype=np.float32)
    d = x.shape[-1]
    assert d % NVFP4_BLOCK == 0
    global_amax = np.maximum(np.abs(x).max(), np.float32(1e-12)).astype(np.float32)
    scale = float(np.float32(global_amax / np.float32(E2M1_MAX * E4M3_MAX)))
    blocks = x.reshape(*x.shape[:-1], d // NVFP4_BLOCK, NVFP4_BLOCK)
    block_amax = np.maximum(np.abs(blocks).max(axis=-1, keepdims=True), np.float32(1e-12)).astype(np.float32)
    micro_f = ((block_amax / np.float32(E2M1_MAX)).astype(np.float32) / np.float32(scale)).astype(np.float32)
    micro_u8 = e4m3_encode(micro_f)
    eff_micro = (e4m3_decode(micro_u8) * np.float32(scale)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        y = (blocks / eff_micro).astype(np.float32)
    ay = np.abs(y)
    mag_idx = np.searchsorted(E2M1_MIDPOINTS, ay.ravel(), side="left").reshape(ay.shape).astype(np.uint8)
    sign = (y < 0).astype(np.uint8)
    code = ((sign << 3) | mag_idx).reshape(*x.shape[:-1], d // 2, 2)
    packed = (code[..., 0] | (code[..., 1] << 4)).astype(np.uint8)
    return packed, micro_u8[..., 0], scale


def dequantize_nvfp4(packed_u8, micro_u8, scale):
    """fa_kernels/paged.py:173-189."""
    packed_u8 = np.asarray(packed_u8, dtype=np.uint8)
    d = packed_u8.shape[-1] * 2
    lo = packed_u8 & 0xF
    hi = packed_u8 >> 4
    code = np.stack([lo, hi], axis=-1).reshape(*packed_u8.shape[:-1], d)
    mag = E2M1_LEVELS[(code & 0x7).astype(np.int64)]
    sign = ((code >> 3) & 1).astype(np.float32)
    e2m1 = mag * (np.float32(1.0) - np.float32(2.0) * sign)
    micro = (e4m3_decode(micro_u8) * np.float32(scale)).astype(np.float32)
    micro = np.repeat(micro, NVFP4_BLOCK, axis=-1)
    return (e2m1 * micro).astype(np.float32)


# ----------------------------------------------------------------------------------------------
# Paged layout — fa_kernels/paged.py:48-91.  `perm` is passed in explicitly: the reference draws it
# from a torch generator on the input's device, and CPU and CUDA generators give different
# permutations, so a bit-exact comparison must feed the same table to both sides.
# ----------------------------------------------------------------------------------------------
def paged_scatter(x, page_size, perm):
    """[B,H,N_k,dx] -> pool [B*n_logical, page_size, H, dx] with pool[perm[i]] = logical block i
    (zero padded tail).  fa_kernels/paged.py:75-88."""
    x = np.asarray(x)
    B, H, N_k, dx = x.shape
    n_logical = (N_k + page_size - 1) // page_size
    pad = n_logical * page_size - N_k
    xp = np.pad(x, ((0, 0), (0, 0), (0, pad), (0, 0)))
    logical = (xp.reshape(B, H, n_logical, page_size, dx).transpose(0, 2, 3, 1, 4)
                 .reshape(B * n_logical, page_size, H, dx))
    pool = np.empty_like(logical)
    pool[np.asarray(perm, dtype=np.int64)] = logical
    return pool


def build_paged_kv(k, v, page_size, perm):
    """fa_kernels/paged.py:48-91 with the permutation supplied by the caller."""
    B, H, N_k, _ = np.asarray(k).shape
    n_logical = (N_k + page_size - 1) // page_size
    block_table = np.asarray(perm, dtype=np.int64).reshape(B, n_logical).astype(np.int32)
    return paged_scatter(k, page_size, perm), paged_scatter(v, page_size, perm), block_table, N_k


def paged_gather(pool, block_table_row, page_size, n_k):
    """Logical token j of a sequence lives at pool[bt[j // page], j % page] — the kernel gather of
    kernels/v7_paged/paged_attention.cu:118-131.  Returns [H, n_k, dx]."""
    pool = np.asarray(pool)
    j = np.arange(n_k)
    pb = np.asarray(block_table_row, dtype=np.int64)[j // page_size]
    rows = pool[pb, j % page_size]                    # [n_k, H, dx]
    return rows.transpose(1, 0, 2)


# ----------------------------------------------------------------------------------------------
# Attention references.  The reference calls torch SDPA (fa_kernels/reference.py:24,43) or spells
# out matmul/softmax (reference.py:100-111, 155-166); this is the spelled-out form in float64 with
# the log-sum-exp returned alongside (no reference backend returns LSE).
# ----------------------------------------------------------------------------------------------
def attention_ref(q, k, v, *, causal=False, scale=None, q_offset=0, return_lse=False):
    """softmax(scale * q k^T + mask) v for [B,H,N_q,d] x [B,H,N_k,d].

    Mask: key j is excluded when j > i + q_offset (kernels/v7_paged/paged_attention.cu:138); with
    q_offset = 0 and N_q == N_k that is the top-left causal mask of reference.py:160-163.  A row with
    every key masked returns zeros and LSE = -inf (merge kernels' `inv = 0 if l == 0`,
    kernels/v8_gqa_ss/gqa_ss_attention.cu:223).
    """
    qd, kd, vd = (np.asarray(t, dtype=np.float64) for t in (q, k, v))
    d = qd.shape[-1]
    s = scale if scale is not None else 1.0 / (d ** 0.5)
    scores = np.matmul(qd, np.swapaxes(kd, -1, -2)) * s
    if causal:
        n_q, n_k = scores.shape[-2], scores.shape[-1]
        i = np.arange(n_q)[:, None]
        j = np.arange(n_k)[None, :]
        scores = np.where(j > i + q_offset, -np.inf, scores)
    m = scores.max(axis=-1, keepdims=True) if scores.shape[-1] else np.full(scores.shape[:-1] + (1,), -np.inf)
    m_safe = np.where(np.isfinite(m), m, 0.0)
    p = np.exp(scores - m_safe)
    l = p.sum(axis=-1, keepdims=True)
    out = np.matmul(p, vd) / np.where(l > 0, l, 1.0)
    out = np.where(l > 0, out, 0.0)
    if return_lse:
        with np.errstate(divide="ignore"):
            lse = (m_safe + np.log(l))[..., 0]
        return out, np.where(l[..., 0] > 0, lse, -np.inf)
    return out


def gqa_attention_ref(q, k, v, *, causal=False, scale=None, q_offset=0, return_lse=False):
    """fa_kernels/reference.py:27-43 — KV head h_kv serves query heads [h_kv*G, h_kv*G+G)
    (repeat_interleave, not tile)."""
    H_q, H_kv = np.asarray(q).shape[1], np.asarray(k).shape[1]
    if H_kv != H_q:
        assert H_q % H_kv == 0
        G = H_q // H_kv
        k = np.repeat(np.asarray(k), G, axis=1)
        v = np.repeat(np.asarray(v), G, axis=1)
    return attention_ref(q, k, v, causal=causal, scale=scale, q_offset=q_offset, return_lse=return_lse)


def paged_gqa_attention_ref(q, k_pool, v_pool, block_table, page_size, n_k, *, scale=None,
                            causal=False, q_offset=0, return_lse=False, dequant_k=None, dequant_v=None):
    """Paged GQA attention through the block table, one sequence at a time so `n_k` may be a scalar
    (reference contract, fa_kernels/paged.py:379-402) or one length per sequence.

    `dequant_k / dequant_v` map a gathered [H_kv, n, dx] slice of stored bytes to float values (for
    FP8 / NVFP4 pools) — the "apples-to-apples" oracles of reference.py:46-81 dequantise the same
    stored bytes the kernel reads.
    """
    q = np.asarray(q)
    B, H_q, N_q, d = q.shape
    lens = np.broadcast_to(np.asarray(n_k, dtype=np.int64), (B,))
    outs, lses = [], []
    for b in range(B):
        n = int(lens[b])
        kb = paged_gather(k_pool, block_table[b], page_size, n)
        vb = paged_gather(v_pool, block_table[b], page_size, n)
        if dequant_k is not None:
            kb = dequant_k(kb, b)
        if dequant_v is not None:
            vb = dequant_v(vb, b)
        if n == 0:
            o = np.zeros((1, H_q, N_q, vb.shape[-1]))
            l = np.full((1, H_q, N_q), -np.inf)
        else:
            o, l = gqa_attention_ref(q[b:b + 1], kb[None], vb[None], causal=causal, scale=scale,
                                     q_offset=q_offset, return_lse=True)
        outs.append(o)
        lses.append(l)
    out, lse = np.concatenate(outs, 0), np.concatenate(lses, 0)
    return (out, lse) if return_lse else out


def mla_attention_ref(q_absorbed, latent, kv_lora_rank, *, causal=False, scale=None, q_offset=0,
                      return_lse=False):
    """MQA over one shared latent in the latent basis — fa_kernels/reference.py:84-111 with the
    dequantisation left to the caller: `latent` is the already-dequantised operand [B,1,N_k,DQK].
    Scores span all DQK dims, values are the first `kv_lora_rank` dims of the same latent."""
    q_absorbed = np.asarray(q_absorbed)
    latent = np.asarray(latent)
    H_q = q_absorbed.shape[1]
    k = np.repeat(latent, H_q, axis=1)
    v = k[..., :kv_lora_rank]
    DQK = q_absorbed.shape[-1]
    s = scale if scale is not None else 1.0 / (DQK ** 0.5)
    return attention_ref(q_absorbed, k, v, causal=causal, scale=s, q_offset=q_offset, return_lse=return_lse)


def merge_partials_ref(o_parts, lse_parts):
    """Combine normalised partial outputs of disjoint key ranges: the merge algebra of
    kernels/v8_gqa_ss/gqa_ss_attention.cu:209-231 with (m, l) folded into LSE = m + log l.
    o_parts [S, ..., d], lse_parts [S, ...] -> (O [..., d], LSE [...])."""
    o_parts = np.asarray(o_parts, dtype=np.float64)
    lse_parts = np.asarray(lse_parts, dtype=np.float64)
    m = lse_parts.max(axis=0)
    m_safe = np.where(np.isfinite(m), m, 0.0)
    w = np.exp(lse_parts - m_safe)                  # exp(-inf) = 0 for empty ranges
    l = w.sum(axis=0)
    o = (w[..., None] * o_parts).sum(axis=0) / np.where(l > 0, l, 1.0)[..., None]
    o = np.where((l > 0)[..., None], o, 0.0)
    with np.errstate(divide="ignore"):
        lse = np.where(l > 0, m_safe + np.log(l), -np.inf)
    return o, lse


# ----------------------------------------------------------------------------------------------
# NVFP4 scale-granularity study — fa_kernels/nvfp4_recipes.py:31-142 (pinned by no reference test;
# pinned here by goldens generated from the imported module).
# ----------------------------------------------------------------------------------------------
def round_e2m1(y):
    """fa_kernels/nvfp4_recipes.py:31-39."""
    y = np.asarray(y, dtype=np.float32)
    idx = np.searchsorted(E2M1_MIDPOINTS, np.abs(y).ravel(), side="left").reshape(y.shape)
    return np.sign(y) * E2M1_LEVELS[idx]


def fake_quant_nvfp4(x, granularity="block16", *, e4m3_scale=True):
    """fa_kernels/nvfp4_recipes.py:42-73."""
    x = np.asarray(x, dtype=np.float32)
    if granularity == "block16":
        return dequantize_nvfp4(*quantize_nvfp4(x))
    if granularity == "tensor":
        amax = np.abs(x).max()
    elif granularity == "channel":
        amax = np.abs(x).max(axis=tuple(range(x.ndim - 1)), keepdims=True)
    elif granularity == "token":
        amax = np.abs(x).max(axis=-1, keepdims=True)
    else:
        raise ValueError(f"unknown granularity {granularity!r}")
    scale = np.maximum((amax / np.float32(E2M1_MAX)).astype(np.float32), np.float32(1e-12))
    if e4m3_scale:
        scale = np.maximum(e4m3_decode(e4m3_encode(scale)), np.float32(1e-12))
    return (round_e2m1((x / scale).astype(np.float32)) * scale).astype(np.float32)


def attn_rmse(q, k, v, *, k_gran, v_gran, causal=False):
    """fa_kernels/nvfp4_recipes.py:76-87."""
    out_q = gqa_attention_ref(q, fake_quant_nvfp4(k, k_gran), fake_quant_nvfp4(v, v_gran), causal=causal)
    out_ref = gqa_attention_ref(q, k, v, causal=causal)
    return float(np.sqrt(np.mean((out_q - out_ref) ** 2)))


def fp8_attn_rmse(q, k, v, *, causal=False):
    """fa_kernels/nvfp4_recipes.py:90-102."""
    kq = dequantize_fp8_e4m3(*quantize_fp8_e4m3(k))
    vq = dequantize_fp8_e4m3(*quantize_fp8_e4m3(v))
    out_q = gqa_attention_ref(q, kq, vq, causal=causal)
    out_ref = gqa_attention_ref(q, k, v, causal=causal)
    return float(np.sqrt(np.mean((out_q - out_ref) ** 2)))


def fp4_score_collapse_rmse(q, k, v, *, causal=False):
    """fa_kernels/nvfp4_recipes.py:105-142: output RMSE against exact attention of (a) K quantised per
    channel and V per token with exact softmax weights, (b) the same with the softmax weights themselves
    quantised per query row (token granularity) and renormalised.  fp32 arithmetic as in the reference."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    G = q.shape[1] // k.shape[1]
    expand = (lambda x: np.repeat(x, G, axis=1)) if G > 1 else (lambda x: x)
    scale = np.float32(1.0 / np.sqrt(q.shape[-1]))
    n_q, n_k = q.shape[2], k.shape[2]
    mask = np.triu(np.ones((n_q, n_k), dtype=bool), k=1) if causal else None

    def softmax_rows(scores):
        if mask is not None:
            scores = np.where(mask, -np.inf, scores)
        e = np.exp(scores - scores.max(axis=-1, keepdims=True))
        return (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)

    ke, ve = expand(k), expand(v)
    out_ref = np.matmul(softmax_rows(np.matmul(q, ke.transpose(0, 1, 3, 2)) * scale), ve)
    kq = expand(fake_quant_nvfp4(k, "channel"))
    vq = expand(fake_quant_nvfp4(v, "token"))
    p_kv = softmax_rows(np.matmul(q, kq.transpose(0, 1, 3, 2)) * scale)
    out_kv = np.matmul(p_kv, vq)
    p_q = fake_quant_nvfp4(p_kv, "token")
    p_q = p_q / np.maximum(p_q.sum(axis=-1, keepdims=True), np.float32(1e-12))
    out_pq = np.matmul(p_q, vq)

    def rmse(a, b):
        return float(np.sqrt(np.mean((a.astype(np.float64) - b.astype(np.float64)) ** 2)))

    return {"fp4_kv_only": rmse(out_kv, out_ref), "fp4_kv_and_p": rmse(out_pq, out_ref)}
