"""Sampler settings, with the reference's names, meanings and defaults
(src/sample.rs:22-35: temp 0 = greedy, top_p 0.95, top_k 0 = off, repeat_penalty 1.0
over the last 64 tokens)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temp: float = 0.0
    top_p: float = 0.95
    top_k: int = 0
    repeat_penalty: float = 1.0
    repeat_window: int = 64
    seed: int = 0

    def validate(self) -> "SamplingParams":
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if self.repeat_penalty <= 0:
            raise ValueError("repeat_penalty must be positive")
        if self.repeat_window < 0:
            raise ValueError("repeat_window must be >= 0")
        return self

    @property
    def greedy(self) -> bool:
        return self.temp <= 0.0
