"""Sampling options, with the names and meanings of sdcb/HyMT2Sharp's SamplingParams
(src/HyMT2Sharp/Sampling.cs:10-34)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0      # 0 (or below) = greedy argmax, bypasses every other field but the penalty
    top_k: int = 0                # keep the k highest logits; 0 = whole vocabulary
    top_p: float = 1.0            # nucleus cutoff on sorted cumulative probability; 1 = off
    min_p: float = 0.0            # drop candidates below min_p * (highest probability); 0 = off
    repeat_penalty: float = 1.0   # penalty over the last `penalty_window` tokens; 1 = off
    penalty_window: int = 64
    seed: int | None = None       # fixed seed of the random stream; None = from the system's entropy

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def needs_filter(self) -> bool:
        penalised = self.repeat_penalty != 1.0 and self.penalty_window > 0
        return penalised or (not self.greedy and (self.top_k > 0 or self.top_p < 1.0 or self.min_p > 0.0))

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not (self.repeat_penalty > 0):
            raise ValueError("repeat_penalty must be > 0")
        if self.penalty_window < 0:
            raise ValueError("penalty_window must be >= 0")


GREEDY = SamplingParams(temperature=0.0)
