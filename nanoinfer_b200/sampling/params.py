"""Per-request sampling parameters, with the reference's names, meanings and defaults
(include/nanoinfer/sampler/sampling_params.h:25-79)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    """temperature: 1.0 = unscaled, <= 0 = greedy arg-max.  top_k: -1 = off, > 0 keeps the k
    largest logits.  top_p: 1.0 = off, in (0, 1) keeps the smallest set of most probable
    tokens whose mass exceeds p.  repetition_penalty: 1.0 = off; > 1 divides positive and
    multiplies negative logits of tokens already generated.  seed: -1 = a fresh random seed
    per request, >= 0 = reproducible."""
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: int = -1

    def use_greedy(self) -> bool:
        return self.temperature <= 0.0

    def use_top_k(self) -> bool:
        return self.top_k > 0

    def use_top_p(self) -> bool:
        return 0.0 < self.top_p < 1.0

    def use_repetition_penalty(self) -> bool:
        return self.repetition_penalty != 1.0

    @staticmethod
    def greedy() -> "SamplingParams":
        return SamplingParams(temperature=0.0)

    def validate(self) -> None:
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be positive")
        if not self.top_p > 0.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.seed < -1:
            raise ValueError("seed must be -1 (random) or non-negative")
