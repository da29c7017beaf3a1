"""Failures are made visible on the host: every kernel records what it could not do in a device status
word, `fa_kernels.check_status()` reads it, and the host-buffer entry point refuses a bad block table
before anything is launched.  No test here faults or hangs the GPU: a bad table entry is masked by the
kernel, and the one timed-out wait is a self-test kernel waiting a millisecond on a barrier of its own."""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

from helpers import assert_close, dev, paged_varlen, randn
from oracle import fa_oracle as O

pytestmark = pytest.mark.gpu


def _small_decode_case(seed=5):
    lens = [300, 45, 129]
    page, H_kv, G, d = 16, 2, 4, 128
    q_t, q = randn((len(lens), H_kv * G, 1, d), seed)
    ks = [randn((H_kv, n, d), seed * 10 + i)[1] for i, n in enumerate(lens)]
    vs = [randn((H_kv, n, d), seed * 10 + 50 + i)[1] for i, n in enumerate(lens)]
    k_pool, bt, _ = paged_varlen([k.astype(np.float16) for k in ks], page, seed)
    v_pool, _, _ = paged_varlen([v.astype(np.float16) for v in vs], page, seed)
    ref = np.concatenate([O.gqa_attention_ref(q[b:b + 1], ks[b][None], vs[b][None]) for b in range(len(lens))], 0)
    return q_t, q, dev(k_pool), dev(v_pool), bt, lens, page, ref


def test_bad_block_table_entry_is_masked_flagged_and_cleared():
    from fa_kernels import check_status, gqa_attention, read_status
    q_t, q, k_pool, v_pool, bt, lens, page, ref = _small_decode_case()
    check_status()
    good = gqa_attention(q_t.cuda(), k_pool, v_pool, dev(bt), page, lens)
    assert_close(good, ref, what="decode before the bad table")
    assert read_status() == 0
    bad = bt.copy()
    bad[0, 3] = k_pool.shape[0] + 7            # a page of sequence 0 that does not exist
    out = gqa_attention(q_t.cuda(), k_pool, v_pool, dev(bad), page, lens)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()           # the page was masked, nothing was read from outside the pool
    assert read_status() & 0x10000
    with pytest.raises(RuntimeError, match="block-table entry"):
        check_status()
    assert read_status() == 0                  # cleared by the check
    again = gqa_attention(q_t.cuda(), k_pool, v_pool, dev(bt), page, lens)
    assert_close(again, ref, what="decode after the flag was cleared")
    check_status()


def test_status_checks_after_every_call_when_enabled():
    from fa_kernels import gqa_attention, set_status_checks
    q_t, q, k_pool, v_pool, bt, lens, page, ref = _small_decode_case(6)
    bad = bt.copy()
    bad[1, 0] = -1
    old = set_status_checks(True)
    try:
        with pytest.raises(RuntimeError, match="block-table entry"):
            gqa_attention(q_t.cuda(), k_pool, v_pool, dev(bad), page, lens)
        assert_close(gqa_attention(q_t.cuda(), k_pool, v_pool, dev(bt), page, lens), ref, what="checked call")
    finally:
        set_status_checks(old)


def test_host_buffer_step_refuses_a_bad_table_before_any_launch():
    from fa_kernels import HostDecodeStep, check_status
    q_t, q, k_pool, v_pool, bt, lens, page, ref = _small_decode_case(7)
    B, H_q, N_q, d = q_t.shape
    step = HostDecodeStep(k_pool, v_pool, page, B, H_q, N_q, d, bt.shape[1], out_dtype=torch.float32)
    q_host, out_host = q_t.pin_memory(), torch.full((B, H_q, N_q, d), float("nan")).pin_memory()
    lens_host = torch.tensor(lens, dtype=torch.int32).pin_memory()
    bad = torch.from_numpy(bt.copy())
    bad[2, 1] = k_pool.shape[0]
    with pytest.raises(RuntimeError, match=r"block_table\[2\]\[1\]"):
        step(q_host, bad.pin_memory(), lens_host, out_host)
    torch.cuda.synchronize()
    assert torch.isnan(out_host).all()          # nothing ran
    step(q_host, torch.from_numpy(bt).pin_memory(), lens_host, out_host)
    torch.cuda.synchronize()
    assert_close(out_host, ref, what="host step after the refused call")
    check_status()


def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_correct():
    """The bounded wait every tcgen05 pipeline uses, on a barrier nothing arrives on: it gives up after its
    bound (here 2 million cycles, about a millisecond), the code lands in a registered status word, the
    host check names it, and the library keeps working afterwards."""
    from fa_kernels import _lib, _status, attention, check_status
    lib = _lib.load()
    check_status()
    word = torch.zeros(4, dtype=torch.int32, device="cuda")
    gave_up = torch.zeros(1, dtype=torch.int32, device="cuda")
    _status.register(word)
    _lib.check(lib.fa_selftest_bounded_wait(word.data_ptr(), 2_000_000, 24, gave_up.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream), "fa_selftest_bounded_wait")
    torch.cuda.synchronize()
    assert int(gave_up.item()) == 1 and int(word[0].item()) == 24
    with pytest.raises(RuntimeError, match="wait for the scores timed out"):
        check_status()
    assert int(word[0].item()) == 0
    q_t, q = randn((1, 2, 200, 64), 3)
    k_t, k = randn((1, 2, 200, 64), 4)
    v_t, v = randn((1, 2, 200, 64), 5)
    assert_close(attention(q_t.cuda(), k_t.cuda(), v_t.cuda(), causal=True), O.attention_ref(q, k, v, causal=True), what="after the timeout")
    check_status()
