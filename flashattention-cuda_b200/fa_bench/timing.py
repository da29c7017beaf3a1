"""CUDA-event timing with an L2 flush before every sample.

Follows the reference's `time_ms_l2flush` (bench/regime.py:114-136): a buffer of at least twice the
L2 size is overwritten outside the event window so that every sample starts from a cold L2 (and a second
buffer is read, so that the cold L2 is also a clean one), and each sample is bracketed by events on the
launching stream.
"""

from __future__ import annotations

import statistics

import torch

_L2_FLUSH_BYTES = 512 << 20   # B200 L2 is ~126 MB; 512 MB leaves nothing resident
_L2_SWEEP_BYTES = 256 << 20   # read afterwards: replaces the dirty lines of the overwrite by clean ones
_flush_buf: dict = {}


def flush_l2(device) -> None:
    """Overwrite 512 MB (nothing of the workload stays in the L2), then read 256 MB of another buffer.
    Without the read the L2 is left full of dirty lines of the flush buffer, and their write-back to HBM
    runs during the first ~20 us of the timed kernel (measured on the paged decode: 222 us after the
    overwrite alone, 211 us after overwrite + read, 212 us under ncu, which starts from an invalidated L2)."""
    bufs = _flush_buf.get(str(device))
    if bufs is None:
        bufs = (torch.empty(_L2_FLUSH_BYTES, dtype=torch.uint8, device=device),
                torch.zeros(_L2_SWEEP_BYTES // 8, dtype=torch.int64, device=device),
                torch.empty(1, dtype=torch.int64, device=device))
        _flush_buf[str(device)] = bufs
    buf, sweep, sink = bufs
    buf.zero_()
    torch.sum(sweep, dim=0, keepdim=True, out=sink)


_SPIN_CYCLES = 600_000        # ~0.3 ms of a kernel that touches no memory


def hold_gpu(device) -> None:
    """Keep the stream busy for ~0.3 ms without touching the L2.  Enqueued after the flush and before the
    start event, it gives the host time to enqueue the timed launch (Python argument handling, plan-cache
    lookup, ctypes call) while the GPU is still working, so that the event window holds the kernel alone
    and no host gap: the start event's timestamp is taken when the spin ends and the timed kernel is
    already queued behind it."""
    torch.cuda._sleep(_SPIN_CYCLES)


def time_cuda(fn, *, warmup: int = 3, iters: int = 10, flush: bool = True, device=None, hold: bool = True):
    """Run `fn` warmup + iters times; return the list of per-iteration milliseconds (CUDA events on the
    current stream around each call, L2 flushed before it, host launch latency kept out of the window)."""
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
        if hold:
            hold_gpu(device)
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return times


def summary(times):
    """Median with the spread: p10 / p50 / p90 / min / max / mean of a list of milliseconds."""
    s = sorted(times)
    n = len(s)

    def pct(p):
        return s[min(n - 1, max(0, int(round(p * (n - 1)))))]
    return {"p50": statistics.median(s), "p10": pct(0.10), "p90": pct(0.90), "min": s[0], "max": s[-1],
            "mean": sum(s) / n, "n": n}
