"""Helpers shared by the GPU parity tests: seeded inputs, paging through the oracle, comparisons."""

from __future__ import annotations

import numpy as np
import torch

from oracle import fa_oracle as O

# fp16 / bf16 outputs must match the fp32-or-better oracle within max-abs 2e-3 and rel 1e-2
ATOL, RTOL = 2e-3, 1e-2


def assert_close(out, ref, atol=ATOL, rtol=RTOL, what=""):
    out = np.asarray(out.detach().float().cpu().numpy() if isinstance(out, torch.Tensor) else out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert out.shape == ref.shape, f"{what}: shape {out.shape} vs {ref.shape}"
    assert np.isfinite(out).all(), f"{what}: non-finite output"
    err = np.abs(out - ref)
    bad = err > atol + rtol * np.abs(ref)
    assert not bad.any(), f"{what}: {bad.sum()} / {bad.size} outside tolerance, max abs err {err.max():.3e}"


def randn(shape, seed, dtype=torch.float16, scale=1.0):
    """Seeded N(0,1)*scale on the CPU generator, rounded to `dtype`; returns (torch tensor, float64 numpy
    of the rounded values) so kernel and oracle read identical numbers."""
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(*shape, generator=g) * scale).to(dtype)
    return x, x.float().numpy().astype(np.float64)


def perm_for(total_blocks, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randperm(total_blocks, generator=g).numpy()


def page(x_np, page_size, perm):
    """[B,H,N,dx] -> pool through the oracle's pager (bit-exact with the reference pager)."""
    return O.paged_scatter(x_np, page_size, perm)


def paged_varlen(per_seq, page_size, seed, n_logical=None):
    """Page sequences of different lengths into one pool.  per_seq: list of [H, n_b, dx] arrays.
    Returns (pool [num_blocks,page,H,dx], block_table [B,n_logical], perm)."""
    B = len(per_seq)
    H, dx = per_seq[0].shape[0], per_seq[0].shape[2]
    n_pages = [max((a.shape[1] + page_size - 1) // page_size, 0) for a in per_seq]
    n_logical = n_logical or max(max(n_pages), 1)
    total = sum(n_pages)
    perm = perm_for(max(total, 1), seed)
    pool = np.zeros((max(total, 1), page_size, H, dx), dtype=per_seq[0].dtype)
    bt = np.zeros((B, n_logical), dtype=np.int32)
    cur = 0
    for b, a in enumerate(per_seq):
        n = a.shape[1]
        for lp in range(n_pages[b]):
            pb = int(perm[cur]); cur += 1
            bt[b, lp] = pb
            rows = a[:, lp * page_size:(lp + 1) * page_size]          # [H, r, dx]
            pool[pb, :rows.shape[1]] = rows.transpose(1, 0, 2)
    return pool, bt, perm


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()
