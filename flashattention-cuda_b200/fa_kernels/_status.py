"""Host side of the device status words.

Every kernel of the library records what it could not do in one int32 of device memory instead of
faulting or hanging: a block-table entry outside the pool (the page is masked and bit 16 is set) or a
bounded pipeline wait that gave up (a code in the low bits).  Nothing on the device reads that word, so
the host has to: `check_status()` synchronises, reads the words of the buffers this process has used on a
device, clears them (and the arrival counters that may have been left behind) and raises RuntimeError
naming the condition.  `set_status_checks(True)` makes every attention call do that before it returns,
which costs a device synchronisation per call and is meant for bring-up and tests.

The reference has no counterpart: its host functions check shapes and dtypes (TORCH_CHECKs,
kernels/v8_gqa_ss/gqa_ss_attention.cu:267-291) and its kernels follow whatever the block table holds.
"""

from __future__ import annotations

import weakref

_enabled = False
_buffers: dict = {}     # device string -> list of weak references to int32 tensors whose word 0 is a status word


def set_status_checks(enabled: bool) -> bool:
    """Check the device status word after every attention call (synchronises).  Returns the old setting."""
    global _enabled
    old, _enabled = _enabled, bool(enabled)
    return old


def status_checks_enabled() -> bool:
    return _enabled


def register(buf) -> None:
    """Remember an int32 CUDA tensor whose element 0 is a status word (idempotent)."""
    refs = _buffers.setdefault(str(buf.device), [])
    for r in refs:
        if r() is buf:
            return
    refs.append(weakref.ref(buf))


def read_status(device=None) -> int:
    """OR of the status words used on `device` so far (synchronises the device; clears nothing)."""
    import torch
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    torch.cuda.synchronize(device)
    word = 0
    alive = []
    for r in _buffers.get(str(device), []):
        buf = r()
        if buf is None:
            continue
        alive.append(r)
        word |= int(buf[0].item())
    _buffers[str(device)] = alive
    return word


def check_status(device=None) -> None:
    """Raise RuntimeError if any kernel launched on `device` recorded an error since the last check.
    The status words and the arrival counters behind them are zeroed first, so the next call starts
    clean."""
    import torch

    from . import _lib
    word = read_status(device)
    if word == 0:
        return
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    for r in _buffers.get(str(device), []):
        buf = r()
        if buf is not None:
            buf.zero_()
    torch.cuda.synchronize(device)
    lib = _lib.load()
    raise RuntimeError("device status: " + lib.fa_status_text(int(word)).decode("utf-8", "replace"))


def after_call(device) -> None:
    if _enabled:
        check_status(device)
