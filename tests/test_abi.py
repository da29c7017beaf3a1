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
        (None, 1048576, 8, 4, 64, -148), ([100, 128, 129, 1000, 9001], 0, 2, 4, 64, -148),      # one CTA per SM (tcgen05 decode)
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


def test_planner_ranges_never_exceed_what_the_kernels_stage():
    """A range of n keys may touch n / page + 2 block-table entries; the decode kernel stages at most 2048
    of them, the MLA kernels 2048 (fused) and 512 (CTA pair, through the chunk hint the host passes).
    Lengths around the multiples of the longest range are where an off-by-one would show."""
    from fa_kernels import _lib
    lib = _lib.load()
    for page in (16, 64, 128, 256):
        longest = 2046 * page
        for ns in (1, 2, 3):
            for delta in (-130, -64, -1, 0, 1, 63, 64, 65, 200):
                n = ns * longest + delta
                if n <= 0:
                    continue
                for B in (1, 4, 64):
                    _, mr = _plan(lib, [n] * B, 0, 8, 4, page, 148)
                    assert mr // page + 2 <= 2048, (page, n, B, mr)
                    _, mr = _plan(lib, [n] * B, 0, 1, 64, page, 148)          # the fused MLA kernel's plan
                    assert mr // page + 2 <= 2048, (page, n, B, mr)
        if page >= 64:
            cap = lib.fa_mla_pair_max_range(page)
            assert cap % 128 == 0 and cap // page + 2 <= 512
            for n in (cap - 1, cap, cap + 1, 2 * cap - 64, 2 * cap + 64, 5 * cap + 1):
                _, mr = _plan(lib, [n, 4096], 0, 1, 64, page, 148, hint=cap)
                assert mr <= cap and mr // page + 2 <= 512, (page, n, mr, cap)
    # the contexts that used to be rejected: 64 sequences of 131008 / 262000 keys at page 64
    for n in (131008, 262000, 130945):
        _, mr = _plan(lib, [n] * 64, 0, 8, 4, 64, 148)
        assert mr // 64 + 2 <= 2048


def test_status_words_have_text():
    from fa_kernels import _lib
    lib = _lib.load()
    assert lib.fa_status_text(0) == b"ok"
    assert b"block-table entry" in lib.fa_status_text(0x10000)
    t = lib.fa_status_text(0x10000 | 47)
    assert b"MLA pair kernel" in t and b"block-table entry" in t
    assert b"dense attention" in lib.fa_status_text(22)
    assert b"timed out" in lib.fa_status_text(999)


def test_roofline_work_counts_match_the_reference_formulas():
    """fa_bench/roofline.py against the numbers the reference's formulas give for the five benchmark
    configurations (roofline/model.py:107-116, 137-142, 197-199) and its three-way bound."""
    import importlib.util
    path = os.path.join(REPO_ROOT, "flashattention-cuda_b200", "fa_bench", "roofline.py")
    spec = importlib.util.spec_from_file_location("fa_roofline", path)
    R = importlib.util.module_from_spec(spec)
    import sys
    sys.modules["fa_roofline"] = R
    spec.loader.exec_module(R)
    w = R.dense_attention(4, 32, 4096, 4096, 128, causal=True)
    assert w.flops == 2 * 4 * 32 * 128 * 4096 * 4097 and abs(w.flops - 5.499e11) < 1e8
    assert R.dense_attention_full_flops(4, 32, 4096, 4096, 128) == 4 * 4 * 32 * 4096 * 4096 * 128
    assert w.total_bytes == 4 * 4 * 32 * 4096 * 128 * 2
    d = R.paged_decode(1000, H_q=32, H_kv=8, d=128)
    assert d.kv_bytes == 4096 * 1000 and d.flops == 4 * 32 * 128 * 1000 and abs(d.flops / d.kv_bytes - 4.0) < 1e-9
    f8 = R.paged_decode(4 * 1048576, H_q=32, H_kv=8, d=128, kv_format="e4m3", per_token_scales=True, B=4)
    assert abs(f8.kv_bytes - 8.858e9) < 1e6
    f4 = R.paged_decode(4 * 1048576, H_q=32, H_kv=8, d=128, kv_format="nvfp4", B=4)
    assert abs(f4.kv_bytes - 4.832e9) < 1e6
    m = R.mla_decode(1000, h_q=128)
    assert m.flops == 278528 * 1000 and m.kv_bytes == 1152 * 1000
    assert R.mla_decode(1000, h_q=128, latent_format="e4m3", per_token_scales=True).kv_bytes == 580 * 1000
    nominal = R.nominal_peaks()
    lb = R.lower_bound(w, nominal)
    assert lb["limiter"] == "mma" and abs(lb["seconds"] - w.flops / 2.25e15) < 1e-12 and abs(lb["ridge"] - 281.25) < 1e-6
    assert R.lower_bound(d, nominal)["limiter"] == "hbm"
    # MLA with a bf16 latent sits just under the ridge (hbm), with an FP8 latent above it (mma)
    assert R.lower_bound(R.mla_decode(128 * 18432, h_q=128, B=128), nominal)["limiter"] == "hbm"
    assert R.lower_bound(R.mla_decode(128 * 18432, h_q=128, latent_format="e4m3", per_token_scales=True, B=128), nominal)["limiter"] == "mma"
    a = R.achieved(d, 1e-6, nominal)
    assert a["bound"] == "hbm" and abs(a["achieved"] - 4096 * 1000 / 1e-6 / 1e9) < 1e-6 and abs(a["frac"] - a["achieved"] / 8000.0) < 1e-12
