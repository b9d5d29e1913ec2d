"""Sampling options, with the reference's names, defaults and meanings
(``GenerationConfig``, crates/mivi-model/src/config.rs:163-195; the sampler's
order of operations, crates/mivi-model/src/sampler.rs:92-136)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

RECENT_TOKENS_WINDOW = 64       # crates/mivi-model/src/config.rs:11


@dataclass
class SamplingParams:
    temperature: float = 0.2            # <= 0: greedy, the first maximum wins
    top_p: float = 0.9                  # >= 1: off
    top_k: int = 40                     # 0: off
    min_p: float = 0.0                  # 0: off
    repetition_penalty: float = 1.05    # 1: off; over the last 64 generated tokens
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: Optional[int] = None          # None: from the clock, as the reference does

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, repetition_penalty=1.0)

    @classmethod
    def plain_temperature(cls, temperature: float, seed: int = 0) -> "SamplingParams":
        """softmax(logits / T) and a categorical draw, nothing else."""
        return cls(temperature=temperature, top_p=1.0, top_k=0, min_p=0.0, repetition_penalty=1.0, seed=seed)

    def validate(self) -> "SamplingParams":
        if self.top_k < 0:
            raise ValueError(f"top_k must be 0 (off) or positive, got {self.top_k}")
        if not (0.0 < self.top_p):
            raise ValueError(f"top_p must be positive, got {self.top_p}")
        if self.min_p < 0.0:
            raise ValueError(f"min_p must not be negative, got {self.min_p}")
        return self

    @property
    def uses_penalties(self) -> bool:
        return ((self.repetition_penalty > 0.0 and self.repetition_penalty != 1.0)
                or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0)
