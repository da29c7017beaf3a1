"""Decode across the GPUs of one box: one process per GPU, `torch.distributed` for the plumbing.

The reference is single-GPU; these are the two ways its decode path shards.

* Batch sharding — every (sequence, KV head) is independent, so ranks own disjoint sequences (and
  their pages and block-table rows).  No collective on the data path; `shard_batch_by_length`
  balances ranks by token count.

* KV-range sharding — one long sequence's keys are cut into contiguous ranges of logical pages, one
  range per rank.  Each rank runs the ordinary decode kernel on its local pool and gets a normalised
  partial output and its log-sum-exp; ONE all-gather of [rows, D + 1] floats per rank moves them, and
  the merge kernel (`fa_merge_partials`, the split-merge algebra of the reference's `*_merge_kernel`,
  kernels/v8_gqa_ss/gqa_ss_attention.cu:209-231) combines them on every rank.  The gathered data is
  only read after NCCL has placed it in local memory.
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple


def shard_batch_by_length(seq_lens: Sequence[int], world: int) -> List[List[int]]:
    """Longest-first greedy assignment of sequences to ranks; returns the sequence indices per rank
    (each list ascending).  Token counts differ by at most the longest sequence."""
    if world < 1:
        raise ValueError("world must be >= 1")
    loads = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for idx in sorted(range(len(seq_lens)), key=lambda i: (-int(seq_lens[i]), i)):
        r = min(range(world), key=lambda j: (loads[j], j))
        owned[r].append(idx)
        loads[r] += int(seq_lens[idx])
    return [sorted(o) for o in owned]


def kv_range_shards(n_k: int, page_size: int, world: int) -> List[Tuple[int, int]]:
    """Cut logical keys [0, n_k) into `world` contiguous page-aligned ranges [(key_begin, key_end)].
    Ranks beyond the last page get an empty range."""
    if world < 1 or page_size < 1 or n_k < 0:
        raise ValueError("bad arguments")
    n_pages = (n_k + page_size - 1) // page_size
    base, extra = divmod(n_pages, world)
    out, page = [], 0
    for r in range(world):
        take = base + (1 if r < extra else 0)
        kb = min(page * page_size, n_k)
        ke = min((page + take) * page_size, n_k)
        out.append((kb, ke))
        page += take
    return out


_exchange: dict = {}


def _exchange_buffers(device, world: int, n_floats: int):
    import torch
    stream = torch.cuda.current_stream(device).cuda_stream if device.type == "cuda" else 0
    key = (str(device), stream, world, n_floats)
    hit = _exchange.get(key)
    if hit is None:
        hit = (torch.empty(n_floats, dtype=torch.float32, device=device),
               torch.empty(world, n_floats, dtype=torch.float32, device=device))
        if len(_exchange) >= 16:
            _exchange.pop(next(iter(_exchange)))
        _exchange[key] = hit
    return hit


def kv_range_decode(attention_fn: Callable, q, args_before_n_k: Sequence, args_after_n_k: Sequence = (), *,
                    local_n_k, key_begin: int, causal: bool = False, q_offset: int = 0, value_dim: Optional[int] = None,
                    group=None, out_dtype=None, return_lse: bool = False, merge_fn: Optional[Callable] = None, **kw):
    """Decode with this rank holding only keys [key_begin, key_begin + local_n_k) of every sequence.

    `attention_fn` is one of this package's paged attention functions, called on the rank-local pools
    and block table as `attention_fn(q, *args_before_n_k, local_n_k, *args_after_n_k, ...)`; e.g. for
    `gqa_attention` args_before_n_k = (k_pool, v_pool, block_table, page_size), for `fp8_attention`
    additionally args_after_n_k = (scale_k, scale_v).  `value_dim` is the output width when it differs
    from q's last dimension (MLA: kv_lora_rank).  Returns the full-context output, identical on every
    rank.  The causal mask is defined on global key positions, so the local call gets
    q_offset - key_begin.
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    B, H_q, N_q = q.shape[0], q.shape[1], q.shape[2]
    D = int(value_dim) if value_dim is not None else q.shape[-1]
    rows = B * H_q * N_q
    # one flat buffer per rank, [rows * D outputs | rows lse], written by the kernel itself, so that a
    # single all-gather moves both; send and receive buffers are kept per (device, stream, shape), so a
    # decode loop allocates nothing here and a captured CUDA graph keeps valid addresses
    send, recv = _exchange_buffers(q.device, world, rows * (D + 1))
    o_loc = send[: rows * D].view(B, H_q, N_q, D)
    lse_loc = send[rows * D:].view(B, H_q, N_q)
    if isinstance(local_n_k, int) and local_n_k == 0:
        o_loc.zero_()                       # no keys here: the neutral element of the merge
        lse_loc.fill_(float("-inf"))
    else:
        attention_fn(q, *args_before_n_k, local_n_k, *args_after_n_k, causal=causal, q_offset=q_offset - key_begin,
                     out_dtype=torch.float32, out=o_loc, lse_out=lse_loc, **kw)
    dist.all_gather_into_tensor(recv.view(-1), send, group=group)
    o_parts = recv[:, : rows * D].unflatten(1, (B, H_q, N_q, D))
    lse_parts = recv[:, rows * D:].unflatten(1, (B, H_q, N_q))
    if merge_fn is None:
        from ._decode import merge_partials as merge_fn
    return merge_fn(o_parts, lse_parts, out_dtype=out_dtype or torch.float32, return_lse=return_lse)
