"""Problem description shared by callers, tests and the benchmark (mirror of the reference's
`AttnConfig`, fa_kernels/config.py:21-58: same fields, same defaults except the target arch)."""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional


@dataclass
class AttnConfig:
    batch: int = 1
    n_heads: int = 8
    seq_len_q: int = 512
    seq_len_k: int = 512
    head_dim: int = 64
    dtype: str = "fp32"
    accum_dtype: str = "fp32"
    causal: bool = False
    scale: Optional[float] = None
    tile_m: Optional[int] = None
    tile_n: Optional[int] = None
    arch: str = "sm_100a"
    layout: str = "BHND"

    def effective_scale(self) -> float:
        return self.scale if self.scale is not None else 1.0 / math.sqrt(self.head_dim)

    def shape(self) -> tuple[int, int, int, int]:
        return (self.batch, self.n_heads, self.seq_len_q, self.head_dim)
