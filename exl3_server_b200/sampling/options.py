"""Sampling options with the reference's names, meanings and defaults
(``SampleOptions``, src/model.h:191-200; flags in src/main.cpp:139-153)."""
from __future__ import annotations

from dataclasses import dataclass

DEFAULT_SEED = 0x9E3779B97F4A7C15   # src/model.h:199
MASK64 = (1 << 64) - 1


@dataclass
class SampleOptions:
    temperature: float = 0.0        # <= 0: greedy
    top_p: float = 1.0
    top_k: int = 0                  # 0: off
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int = DEFAULT_SEED

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def has_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.presence_penalty != 0.0
                or self.frequency_penalty != 0.0)

    @property
    def has_filters(self) -> bool:
        return self.top_k > 0 or self.top_p < 1.0 or self.min_p > 0.0


class SplitMix64:
    """The reference's generator (src/model.cpp:656-665)."""

    def __init__(self, state: int):
        self.state = state & MASK64

    def next(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        return z ^ (z >> 31)

    def uniform01(self) -> float:
        return (self.next() >> 11) * (1.0 / 9007199254740992.0)
