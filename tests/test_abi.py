"""The C-ABI library loads on a CPU-only machine and exports every symbol include/fa_b200.h declares.
No compute entry point is called here."""

from __future__ import annotations

import ctypes as C
import os
import re

from conftest import REPO_ROOT


def _declared():
    text = open(os.path.join(REPO_ROOT, "include", "fa_b200.h")).read()
    return sorted(set(re.findall(r"FA_API\s+[\w\s\*]+?\b(fa_\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    from fa_kernels import _lib
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fa_b200.h but not exported"
    assert lib.fa_version() >= 100


def test_missing_library_is_an_error_not_a_fallback(monkeypatch):
    import importlib
    from fa_kernels import _lib
    monkeypatch.setenv("FA_B200_LIB", "/nonexistent/libfa_b200.so")
    monkeypatch.setattr(_lib, "_lib", None)
    try:
        _lib.load()
        raise AssertionError("load() must raise when the library is absent")
    except RuntimeError as e:
        assert "not found" in str(e)


def test_planner_on_host():
    from fa_kernels import _lib
    lib = _lib.load()
    lens = [1024, 8192, 0, 77, 5000]
    arr = (C.c_int32 * len(lens))(*lens)
    cap = lib.fa_decode_plan_max_items(C.cast(arr, C.c_void_p), 0, len(lens), 16)
    items = (_lib.DecodeItem * cap)()
    n, mr = C.c_int(), C.c_int()
    for hint in (0, 256, 64, 4096):
        assert lib.fa_decode_plan(C.cast(arr, C.c_void_p), 0, len(lens), 8, 4, 16, 148, hint,
                                  C.cast(items, C.c_void_p), cap, C.byref(n), C.byref(mr)) == 0
        got = [items[i] for i in range(n.value)]
        # every sequence is covered exactly once by its ranges, in order of split index
        for b, ln in enumerate(lens):
            mine = sorted((it.split, it.k_begin, it.k_end, it.n_split, it.slot_base) for it in got if it.b == b)
            assert len(mine) == mine[0][3] and [m[0] for m in mine] == list(range(len(mine)))
            assert mine[0][1] == 0 and mine[-1][2] == ln
            assert all(mine[i][2] == mine[i + 1][1] for i in range(len(mine) - 1))
            assert len({m[4] for m in mine}) == 1
        # slots of different sequences do not overlap and ranges come longest first
        slots = sorted((it.slot_base, it.n_split) for it in got if it.split == 0)
        assert all(slots[i][0] + slots[i][1] == slots[i + 1][0] for i in range(len(slots) - 1))
        sizes = [it.k_end - it.k_begin for it in got]
        assert sizes == sorted(sizes, reverse=True) and max(sizes) == mr.value
        assert all((it.k_begin % 64) == 0 for it in got)
    # invalid arguments are reported, not crashed on
    assert lib.fa_decode_plan(None, -5, 1, 1, 1, 16, 148, 0, C.cast(items, C.c_void_p), cap, C.byref(n), C.byref(mr)) == 1
    assert b"negative" in lib.fa_last_error()


def _plan(lib, lens, n_k, H_kv, rows, page, sms, hint=0):
    from fa_kernels import _lib
    B = len(lens) if lens is not None else 4
    arr = (C.c_int32 * B)(*lens) if lens is not None else None
    ptr = C.cast(arr, C.c_void_p) if arr is not None else None
    cap = lib.fa_decode_plan_max_items(ptr, n_k, B, page)
    items = (_lib.DecodeItem * cap)()
    n, mr = C.c_int(), C.c_int()
    assert lib.fa_decode_plan(ptr, n_k, B, H_kv, rows, page, sms, hint, C.cast(items, C.c_void_p), cap,
                              C.byref(n), C.byref(mr)) == 0
    assert n.value <= cap
    return [items[i] for i in range(n.value)], mr.value


def test_planner_candidates_cover_every_sequence_once():
    """The planner picks between whole sequences, two or three equal ranges and shrinking ranges; whatever
    it picks, the ranges of a sequence tile [0, len) in split order, start on multiples of 64, own
    consecutive partial-result slots, and come longest first.  Shapes: one wave of whole sequences, a
    partly filled second wave (equal splits), few long sequences (shrinking ranges), a single head, and
    slot counts given exactly (negative num_sms)."""
    from fa_kernels import _lib
    lib = _lib.load()
    shapes = [
        ([8192] * 37, 0, 8, 4, 16, -296), ([8192] * 45, 0, 8, 4, 16, -296), ([8192] * 80, 0, 8, 4, 16, -296),
        (None, 1048576, 8, 4, 64, 148), ([131072], 0, 1, 1, 256, -296), ([5, 70000, 0, 64, 4097], 0, 2, 16, 16, 148),
        ([300] * 1000, 0, 8, 4, 16, 148),
    ]
    kinds = set()
    for lens, n_k, H_kv, rows, page, sms in shapes:
        got, mr = _plan(lib, lens, n_k, H_kv, rows, page, sms)
        seq = lens if lens is not None else [n_k] * 4
        for b, ln in enumerate(seq):
            mine = sorted((it.split, it.k_begin, it.k_end, it.n_split, it.slot_base) for it in got if it.b == b)
            assert len(mine) == mine[0][3] and [m[0] for m in mine] == list(range(len(mine)))
            assert mine[0][1] == 0 and mine[-1][2] == ln
            assert all(mine[i][2] == mine[i + 1][1] for i in range(len(mine) - 1))
            assert len({m[4] for m in mine}) == 1
        sizes = [it.k_end - it.k_begin for it in got]
        assert sizes == sorted(sizes, reverse=True) and max(sizes) == mr
        assert all((it.k_begin % 64) == 0 for it in got)
        per_seq = len(got) / len(seq)
        kinds.add("whole" if per_seq == 1 else ("few" if per_seq <= 3 else "many"))
    assert kinds == {"whole", "few", "many"}          # each kind of plan was chosen somewhere
    # one full wave of equal sequences stays whole; a wave and a half is cut
    assert len(_plan(lib, [8192] * 37, 0, 8, 4, 16, -296)[0]) == 37
    assert len(_plan(lib, [8192] * 45, 0, 8, 4, 16, -296)[0]) > 45


def test_sweep_takes_the_reference_harness_flags():
    """fa_bench/sweep.py parses the command lines of the reference's bench/harness.py (:357-397) and
    bench/regime.py (:292-320) unchanged."""
    import importlib.util
    path = os.path.join(REPO_ROOT, "flashattention-cuda_b200", "fa_bench", "sweep.py")
    spec = importlib.util.spec_from_file_location("fa_sweep_cli", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    parse = mod.build_parser().parse_args
    a = parse("--backend v8_gqa_ss --precision fp16 --batch-sweep 1 8 16 32 64 --page-size 256 --heads 32 --causal "
              "--seq 8192 --dim 64 128 --decode --q-len 4 --gqa-group 1 2 4 8".split())
    assert a.batch_sweep == [1, 8, 16, 32, 64] and a.gqa_groups == [1, 2, 4, 8] and a.decode and a.q_len == 4
    assert a.seq == [8192] and a.dim == [64, 128] and a.page_size == 256 and a.causal
    b = parse("--backend v12_mla_tc --mla-engine nvfp4 --kv-lens 8192 1048576 --h-kv 1 8 --max-ws-gb 8 --batch 2".split())
    assert b.mla_engine == "nvfp4" and b.seq == [8192, 1048576] and b.h_kvs == [1, 8] and b.max_ws_gb == 8.0 and b.batch == 2
