"""Host-side sharding logic and the all-gather + merge protocol with two gloo ranks on CPU.

The CUDA kernels cannot run here, so the rank-local attention and the merge are the oracle's (injected
through the wrapper's `attention_fn` / `merge_fn` hooks); what is under test is the product's
sharding arithmetic, the q_offset translation, the packing of (O, LSE) into one all-gather and the
view arithmetic that unpacks it."""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_DIR, REPO_ROOT


def test_shard_batch_by_length_balances_tokens():
    from fa_kernels.distributed import shard_batch_by_length
    g = np.random.default_rng(2)
    lens = g.integers(1024, 8193, 64).tolist()
    for world in (1, 2, 4, 8):
        owned = shard_batch_by_length(lens, world)
        assert sorted(i for o in owned for i in o) == list(range(64))
        loads = [sum(lens[i] for i in o) for o in owned]
        assert max(loads) - min(loads) <= max(lens)
    assert shard_batch_by_length([5, 1], 4) == [[0], [1], [], []]


def test_kv_range_shards_cover_once_and_are_page_aligned():
    from fa_kernels.distributed import kv_range_shards
    for n_k, page, world in [(1048576, 64, 8), (1000, 64, 4), (63, 64, 4), (0, 16, 2), (8190, 16, 8), (129, 64, 2)]:
        sh = kv_range_shards(n_k, page, world)
        assert len(sh) == world and sh[0][0] == 0 and sh[-1][1] == n_k
        assert all(a[1] == b[0] for a, b in zip(sh, sh[1:]))
        assert all(kb % page == 0 for kb, ke in sh if ke > kb)
        sizes = [(ke - kb + page - 1) // page for kb, ke in sh]
        assert max(sizes) - min(sizes) <= 1


def _oracle_attention(q, k, v, n_k, *, causal, q_offset, out_dtype, out, lse_out):
    """Stand-in for the CUDA attention on a dense rank-local K/V slice (CPU test only)."""
    from oracle import fa_oracle as O
    o, lse = O.gqa_attention_ref(q.numpy(), k[:, :, :n_k].numpy(), v[:, :, :n_k].numpy(), causal=causal,
                                 q_offset=q_offset, return_lse=True)
    out.copy_(torch.from_numpy(o).float())
    lse_out.copy_(torch.from_numpy(lse).float())


def _oracle_merge(o_parts, lse_parts, out_dtype, return_lse):
    from oracle import fa_oracle as O
    o, lse = O.merge_partials_ref(o_parts.numpy(), lse_parts.numpy())
    o = torch.from_numpy(o).to(out_dtype)
    return (o, torch.from_numpy(lse).float()) if return_lse else o


def _worker(rank, world, port, causal, ret):
    for p in (PKG_DIR, REPO_ROOT):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fa_kernels.distributed import kv_range_decode, kv_range_shards
        from oracle import fa_oracle as O
        g = torch.Generator().manual_seed(7)
        B, H_q, H_kv, N_q, d, page, n_k = 2, 4, 2, 3, 32, 16, 203
        q = torch.randn(B, H_q, N_q, d, generator=g)
        k = torch.randn(B, H_kv, n_k, d, generator=g)
        v = torch.randn(B, H_kv, n_k, d, generator=g)
        q_offset = n_k - N_q
        kb, ke = kv_range_shards(n_k, page, world)[rank]
        out, lse = kv_range_decode(_oracle_attention, q, (k[:, :, kb:ke].contiguous(), v[:, :, kb:ke].contiguous()),
                                   local_n_k=ke - kb, key_begin=kb, causal=causal, q_offset=q_offset,
                                   return_lse=True, merge_fn=_oracle_merge)
        ref, ref_lse = O.gqa_attention_ref(q.numpy(), k.numpy(), v.numpy(), causal=causal, q_offset=q_offset, return_lse=True)
        ok = np.allclose(out.numpy(), ref, atol=1e-5) and np.allclose(lse.numpy(), ref_lse, atol=1e-5)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("world", [2, 3])
def test_kv_range_decode_protocol_on_gloo(world, causal):
    port = 29500 + (os.getpid() + world * 7 + int(causal)) % 2000
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, causal, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def _absent_rank_worker(rank, world, port, ret):
    for p in (PKG_DIR, REPO_ROOT):
        if p not in sys.path:
            sys.path.insert(0, p)
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from fa_kernels.distributed import kv_range_decode, kv_range_shards
    if rank == 1:
        # this rank joined the group but never reaches the step's all-gather (a stalled worker)
        ret[rank] = "absent"
        time.sleep(10.0)
        return
    g = torch.Generator().manual_seed(7)
    B, H_q, H_kv, N_q, d, page, n_k = 1, 2, 1, 1, 16, 16, 64
    q = torch.randn(B, H_q, N_q, d, generator=g)
    k = torch.randn(B, H_kv, n_k, d, generator=g)
    v = torch.randn(B, H_kv, n_k, d, generator=g)
    kb, ke = kv_range_shards(n_k, page, world)[rank]
    t0 = time.time()
    try:
        kv_range_decode(_oracle_attention, q, (k[:, :, kb:ke].contiguous(), v[:, :, kb:ke].contiguous()),
                        local_n_k=ke - kb, key_begin=kb, merge_fn=_oracle_merge)
        ret[rank] = "returned"
    except Exception as exc:                       # the collective's timeout surfaces as a Python exception
        ret[rank] = f"raised {type(exc).__name__} after {time.time() - t0:.1f} s"


def test_a_rank_that_never_joins_the_all_gather_becomes_an_exception():
    """Failure detection on the host: with a process-group timeout, the rank that does reach the all-gather
    of kv_range_decode gets an exception instead of waiting for ever (CPU ranks, gloo)."""
    port = 31500 + os.getpid() % 2000
    ret = mp.Manager().dict()
    ctx = mp.spawn(_absent_rank_worker, args=(2, port, ret), nprocs=2, join=False)
    deadline = 60.0
    import time
    t0 = time.time()
    while time.time() - t0 < deadline and not str(ret.get(0, "")).startswith(("raised", "returned")):
        time.sleep(0.2)
    for p in ctx.processes:
        p.join(timeout=15)
        if p.is_alive():
            p.terminate()
    assert ret.get(1) == "absent"
    assert str(ret.get(0, "")).startswith("raised"), dict(ret)
