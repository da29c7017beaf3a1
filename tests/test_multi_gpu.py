"""KV-range-sharded decode on two real GPUs over NCCL (skipped with fewer than two devices).

Every rank holds half of each sequence's keys in its own paged pool, runs the decode kernel locally,
all-gathers (O, LSE) and merges; the result must equal the oracle on the full context on every rank."""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

from conftest import PKG_DIR, REPO_ROOT

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, fmt, ret):
    for p in (PKG_DIR, REPO_ROOT, os.path.join(REPO_ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from fa_kernels import fp8_attention, gqa_attention
        from fa_kernels.distributed import kv_range_decode, kv_range_shards
        from fa_kernels.paged import build_paged_kv, build_paged_kv_fp8_per_token
        from oracle import fa_oracle as O
        g = torch.Generator().manual_seed(11)
        B, H_q, H_kv, d, page, n_k = 2, 8, 2, 128, 64, 5000
        q = torch.randn(B, H_q, 1, d, generator=g).half()
        k = torch.randn(B, H_kv, n_k, d, generator=g).half()
        v = torch.randn(B, H_kv, n_k, d, generator=g).half()
        kb, ke = kv_range_shards(n_k, page, world)[rank]
        k_loc, v_loc = k[:, :, kb:ke].contiguous().cuda(), v[:, :, kb:ke].contiguous().cuda()
        if fmt == "f16":
            kp, vp, bt, n_loc = build_paged_kv(k_loc, v_loc, page, seed=rank)
            out = kv_range_decode(gqa_attention, q.cuda(), (kp, vp, bt, page), local_n_k=n_loc, key_begin=kb,
                                  causal=True, q_offset=n_k - 1)
            ref = O.gqa_attention_ref(q.float().numpy(), k.float().numpy(), v.float().numpy())
        else:
            kp, vp, bt, n_loc, ks, vs = build_paged_kv_fp8_per_token(k_loc, v_loc, page, seed=rank)
            out = kv_range_decode(fp8_attention, q.cuda(), (kp, vp, bt, page), (ks, vs), local_n_k=n_loc, key_begin=kb)
            kq, ksc = O.quantize_fp8_e4m3_per_token(k.float().numpy())
            vq, vsc = O.quantize_fp8_e4m3_per_token(v.float().numpy())
            ref = O.gqa_attention_ref(q.float().numpy(), O.e4m3_decode(kq) * ksc[..., None], O.e4m3_decode(vq) * vsc[..., None])
        torch.cuda.synchronize()
        err = np.abs(out.cpu().numpy() - ref)
        ret[rank] = bool((err <= 2e-3 + 1e-2 * np.abs(ref)).all())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fmt", ["f16", "e4m3"])
def test_kv_range_decode_over_nccl(fmt):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 1000
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, fmt, ret), nprocs=2, join=True)
    assert ret.get(0) and ret.get(1), dict(ret)


def _batch_worker(rank, world, port, ret):
    for p in (PKG_DIR, REPO_ROOT, os.path.join(REPO_ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from fa_kernels import check_status, gqa_attention
        from fa_kernels.distributed import shard_batch_by_length
        from helpers import dev, paged_varlen, randn
        from oracle import fa_oracle as O
        lens = [5000, 120, 3000, 4097, 64, 2500, 1, 900]
        H_kv, G, d, page = 2, 4, 128, 16
        mine = shard_batch_by_length(lens, world)[rank]
        ks = [randn((H_kv, lens[i], d), 300 + i)[1] for i in mine]          # sequence i has the same values on any rank
        vs = [randn((H_kv, lens[i], d), 400 + i)[1] for i in mine]
        q_t = torch.cat([randn((1, H_kv * G, 1, d), 500 + i)[0] for i in mine])
        k_pool, bt, _ = paged_varlen([k.astype(np.float16) for k in ks], page, 20 + rank)
        v_pool, _, _ = paged_varlen([v.astype(np.float16) for v in vs], page, 20 + rank)
        out = gqa_attention(q_t.cuda(), dev(k_pool), dev(v_pool), dev(bt), page, [lens[i] for i in mine])
        check_status()
        ok = True
        for j, i in enumerate(mine):
            ref = O.gqa_attention_ref(q_t[j:j + 1].float().numpy().astype(np.float64), ks[j][None], vs[j][None])
            err = np.abs(out[j:j + 1].cpu().numpy() - ref)
            ok = ok and bool((err <= 2e-3 + 1e-2 * np.abs(ref)).all())
        # the outputs of all ranks, gathered for the caller: every sequence exactly once
        full = torch.zeros(len(lens), H_kv * G, 1, d, device="cuda")
        full[mine] = out
        dist.all_reduce(full)
        owners = [None] * world
        dist.all_gather_object(owners, mine)
        ok = ok and sorted(i for o in owners for i in o) == list(range(len(lens)))
        ok = ok and bool(torch.equal(full[mine], out)) and bool((full.abs().amax(dim=(1, 2, 3)) > 0).all())
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_batch_sharded_decode_over_nccl():
    """Sequences dealt to two GPUs by token count (no collective on the data path); each rank's outputs match
    the oracle and the gathered batch holds every sequence once."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29700 + os.getpid() % 1000
    ret = mp.Manager().dict()
    mp.spawn(_batch_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret.get(0) and ret.get(1), dict(ret)
