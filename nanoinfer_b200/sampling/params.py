"""Sampling options of a request, with the reference's names, defaults and checks
(nanoinfer/sampling.py:31-55, cpp/src/sampling.cpp:24-31)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 0.0          # 0 = greedy (first index of the maximum)
    top_k: Optional[int] = None       # keep the k largest logits; None or <= 0: off
    top_p: Optional[float] = None     # nucleus; None or >= 1: off
    repetition_penalty: float = 1.0   # 1 = off; > 1 lowers the logits of tokens already seen
    seed: Optional[int] = None        # seeds the draws of this request

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")
        if self.top_p is not None and self.top_p < 0:
            raise ValueError(f"top_p must be >= 0, got {self.top_p}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def k(self) -> int:
        return int(self.top_k) if self.top_k and self.top_k > 0 else 0

    @property
    def p(self) -> float:
        return float(self.top_p) if self.top_p is not None and self.top_p < 1.0 else 1.0
