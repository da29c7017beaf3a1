"""CUDA-event timing with an L2 flush before every sample.

Follows the reference's `time_ms_l2flush` (bench/regime.py:114-136): a buffer of at least twice the
L2 size is overwritten outside the event window so that every sample starts from a cold L2, and
each sample is bracketed by events on the launching stream.
"""

from __future__ import annotations

import statistics

import torch

_L2_FLUSH_BYTES = 512 << 20   # B200 L2 is ~126 MB; 512 MB leaves nothing resident
_flush_buf: dict = {}


def flush_l2(device) -> None:
    buf = _flush_buf.get(str(device))
    if buf is None:
        buf = torch.empty(_L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
        _flush_buf[str(device)] = buf
    buf.zero_()


def time_cuda(fn, *, warmup: int = 3, iters: int = 10, flush: bool = True, device=None):
    """Run `fn` warmup + iters times; return the list of per-iteration milliseconds."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    for _ in range(warmup):
        if flush:
            flush_l2(device)
        fn()
    torch.cuda.synchronize(device)
    times = []
    for _ in range(iters):
        if flush:
            flush_l2(device)
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return times


def summary(times):
    s = sorted(times)
    return {"p50": statistics.median(s), "min": s[0], "max": s[-1], "mean": sum(s) / len(s)}
