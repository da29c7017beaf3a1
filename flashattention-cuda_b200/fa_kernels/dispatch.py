"""Backend name -> operator object with a `.forward(...)`, gated on compute capability.

Same contract as the reference's fa_kernels/dispatch.py:69-80: unknown name -> KeyError, GPU below
the required capability -> RuntimeError, no CUDA device -> RuntimeError.  Every reference backend
name is accepted and maps to the one B200 implementation of its operator family ("b200" names the
family default); all of them need sm_100.
"""

from __future__ import annotations

import torch

from . import _lib

_B200 = (10, 0)

# backend name -> operator family (the positional `forward` signature differs per family,
# kernels/*/binding.cpp)
_FAMILY = {
    "v1_naive": "dense", "v2_tiled": "dense", "v3_online": "dense", "v4_fused": "dense",
    "v5_wmma": "dense", "v6_splitkv": "dense", "b200_dense": "dense",
    "v7_paged": "paged", "v8_gqa": "paged", "v8_gqa_tc": "paged", "v8_gqa_db": "paged",
    "v8_gqa_occ": "paged", "v8_gqa_ilp": "paged", "v8_gqa_ss": "paged", "b200_paged": "paged",
    "v9_fp8": "fp8", "b200_fp8": "fp8",
    "v10_nvfp4": "nvfp4", "b200_nvfp4": "nvfp4",
    "v11_mla": "mla", "b200_mla": "mla",
    "v12_mla_tc": "mla_tc", "b200_mla_tc": "mla_tc",
}
_MIN_CAPABILITY = {name: _B200 for name in _FAMILY}


def _current_capability() -> tuple[int, int]:
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device visible; kernels run on the GPU (B200, sm_100a)")
    return torch.cuda.get_device_capability()


class _Backend:
    """What `build_kernel(name)` returns in the reference: an object whose `.forward` takes the
    family's positional arguments."""

    def __init__(self, name: str, family: str):
        self.name, self.family = name, family

    def forward(self, *args, **kwargs):
        from . import _ops
        return getattr(_ops, f"{self.family}_forward")(*args, **kwargs)

    def __repr__(self):
        return f"<fa_b200 backend {self.name} ({self.family})>"


_cache: dict = {}


def get_backend(name: str):
    """Return the operator for `name`, or raise if this GPU can't run it."""
    if name not in _MIN_CAPABILITY:
        raise KeyError(f"unknown backend {name!r}; known: {sorted(_MIN_CAPABILITY)}")
    need = _MIN_CAPABILITY[name]
    have = _current_capability()
    if have < need:
        raise RuntimeError(
            f"backend {name!r} needs compute capability >= {need[0]}.{need[1]}, "
            f"but this GPU is {have[0]}.{have[1]}")
    _lib.load()                      # fail here, loudly, when the CUDA library is missing
    if name not in _cache:
        _cache[name] = _Backend(name, _FAMILY[name])
    return _cache[name]
