"""fa_paged_decode_fwd_static — the decode entry point that brings its own scratch.

Some hosts of this library cannot allocate device memory: a server that gave the whole GPU to its
KV-cache pool at start-up, or a plugin host that hands over buffers but no allocator.  For them the
library carries a fixed scratch array in its device image.  This test drives that entry point through
the C ABI and checks it against the ordinary entry point (caller-supplied scratch) on the same inputs,
twice in a row, because the second call starts from whatever the first left in the shared array.

Collected last (file name), so that a run that stops at the first failure has already run the others.
"""

from __future__ import annotations

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(q, k_pool, v_pool, bt, page, lens, out, chunk_hint):
    """A fa_decode_args for fp16 pools with per-sequence lengths; scratch fields left empty."""
    from fa_kernels import _decode, _lib
    B, H_q, N_q, d = q.shape
    H_kv = k_pool.shape[2]
    items, n_items, n_slots, max_range, _ = _decode.plan(tuple(lens), max(lens), B, H_kv, (H_q // H_kv) * N_q, page,
                                                         q.device, chunk_hint)
    a = _lib.DecodeArgs()
    a.q, a.q_dtype = q.data_ptr(), _lib.FA_F16
    a.k_pool, a.v_pool, a.kv_dtype = k_pool.data_ptr(), v_pool.data_ptr(), _lib.FA_F16
    a.k_scale = a.v_scale = 1.0
    a.block_table, a.n_logical, a.num_blocks, a.page_size = bt.data_ptr(), bt.shape[1], k_pool.shape[0], page
    a.B, a.H_q, a.H_kv, a.N_q, a.D = B, H_q, H_kv, N_q, d
    a.softmax_scale = 1.0 / d ** 0.5
    a.items, a.n_items, a.n_slots, a.max_range_keys = items.data_ptr(), n_items, n_slots, max_range
    a.out, a.out_dtype = out.data_ptr(), _lib.FA_F32
    a.stream = torch.cuda.current_stream().cuda_stream
    return a, items


def test_static_scratch_entry_point_matches_caller_scratch_twice():
    from fa_kernels import _decode, _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(77)
    B, H_q, H_kv, d, page = 3, 8, 2, 128, 16
    lens = [5000, 777, 2049]
    n_pages = [(n + page - 1) // page for n in lens]
    total = sum(n_pages)
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(B, max(n_pages), dtype=torch.int32)
    cur = 0
    for b, n in enumerate(n_pages):
        bt[b, :n] = perm[cur:cur + n].to(torch.int32)
        cur += n
    bt = bt.to(dev)
    k_pool = torch.randn(total, page, H_kv, d, generator=g).half().to(dev)
    v_pool = torch.randn(total, page, H_kv, d, generator=g).half().to(dev)

    for call, chunk_hint in enumerate((256, 512)):       # both calls split the sequences -> scratch is used
        q = torch.randn(B, H_q, 1, d, generator=g).half().to(dev)
        # existing entry point, scratch supplied by the caller
        want = torch.empty(B, H_q, 1, d, dtype=torch.float32, device=dev)
        a, keep = _args(q, k_pool, v_pool, bt, page, lens, want, chunk_hint)
        assert a.n_slots > B, "the case must exercise split sequences"
        ws, cnt = _decode.workspace(dev, lib.fa_decode_workspace_bytes(a.n_slots, H_q, 1, d),
                                    lib.fa_decode_counters_len(B, H_q, H_kv, 1))
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        a.counters, a.counters_len = cnt.data_ptr(), cnt.numel()
        _lib.check(lib.fa_paged_decode_fwd(C.byref(a)), "fa_paged_decode_fwd")
        # new entry point: no scratch passed at all
        got = torch.full((B, H_q, 1, d), float("nan"), dtype=torch.float32, device=dev)
        s, keep2 = _args(q, k_pool, v_pool, bt, page, lens, got, chunk_hint)
        torch.cuda.synchronize()
        free_before, torch_before = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev)
        _lib.check(lib.fa_paged_decode_fwd_static(C.byref(s)), "fa_paged_decode_fwd_static")
        torch.cuda.synchronize()
        if call == 1:
            # the property the entry point exists for: the call took no device memory, neither from the
            # driver (cudaMemGetInfo) nor from torch's allocator.  (The first call on a device may make the
            # driver load the kernel image, so the second call is the one measured.)
            assert torch.cuda.mem_get_info(dev)[0] == free_before
            assert torch.cuda.memory_allocated(dev) == torch_before
        assert torch.isfinite(got).all(), f"call {call}: output not fully written"
        # same kernel, same plan, same merge order: the two scratch arrangements give identical bits
        assert torch.equal(got, want), f"call {call}: max abs diff {(got - want).abs().max().item():.3e}"
    # and the oracle agrees with both (the comparison above is between two paths of this library)
    from helpers import assert_close
    from oracle import fa_oracle as O
    ref = O.paged_gqa_attention_ref(q.float().cpu().numpy().astype("float64"), k_pool.float().cpu().numpy().astype("float64"),
                                    v_pool.float().cpu().numpy().astype("float64"), bt.cpu().numpy(), page, lens)
    assert_close(got, ref, what="static-scratch decode vs oracle")
    # no kernel of these calls raised a status flag, and the word can be read back and cleared
    word = C.c_int32(-1)
    _lib.check(lib.fa_paged_decode_static_status(C.byref(word), 1, torch.cuda.current_stream().cuda_stream), "static_status")
    assert word.value == 0


def test_static_scratch_rejects_oversized_requests():
    from fa_kernels import _lib
    lib = _lib.load()
    a = _lib.DecodeArgs()
    dummy = torch.zeros(16, device="cuda:0")
    a.q = a.k_pool = a.v_pool = a.block_table = a.items = a.out = dummy.data_ptr()
    a.B, a.H_q, a.H_kv, a.N_q, a.D = 4096, 32, 8, 1, 128       # 32768 units > 16384
    a.n_items, a.n_slots = 4096, 0
    assert lib.fa_paged_decode_fwd_static(C.byref(a)) == 4     # FA_ERR_WORKSPACE
    assert b"built-in" in lib.fa_last_error()
    a.B, a.H_q, a.H_kv, a.n_items = 16385, 1, 1, 16385          # one unit past the documented 16384
    assert lib.fa_paged_decode_fwd_static(C.byref(a)) == 4
    a.B, a.H_q, a.H_kv = 64, 32, 8
    a.n_items = a.n_slots = 1 << 20                             # partial results far beyond 8 MiB
    assert lib.fa_paged_decode_fwd_static(C.byref(a)) == 4
    assert b"built-in" in lib.fa_last_error()
    # a malformed request is an argument error, found before anything touches the shared array
    a.B = -3
    assert lib.fa_paged_decode_fwd_static(C.byref(a)) == 1     # FA_ERR_INVALID
