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
