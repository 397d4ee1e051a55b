"""Sampling options, with the reference's names, meanings and defaults
(src/engine/sampler.rs:9-29): ``temperature`` 0 = greedy (first maximum),
``top_k`` 0 = off, ``top_p`` 1.0 = off, ``seed`` None = 42
(src/engine/generate.rs:672).  The sampling itself is a kernel
(csrc/sampling.cu) fed with the step's 32-bit logits.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DEFAULT_SEED = 42


@dataclass(frozen=True)
class SamplingConfig:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: Optional[int] = None

    def __post_init__(self):
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 < self.top_p:
            raise ValueError(f"top_p must be positive, got {self.top_p}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    def seed_value(self) -> int:
        return DEFAULT_SEED if self.seed is None else int(self.seed)
