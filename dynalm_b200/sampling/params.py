"""Sampling parameters with the reference's names, defaults and ranges
(dynalm/src/sampling/sampler.h:31-48; validation dynalm/src/sampling/sampler.cpp:40-51)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..errors import InvalidArgument


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0          # <= 0: greedy
    top_k: int = 0                    # 0: off; 1: greedy
    top_p: float = 1.0                # 1: off
    min_p: float = 0.0                # 0: off
    repetition_penalty: float = 1.0   # 1: off
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    penalty_last_n: int = 64          # -1: the whole context
    seed: Optional[int] = None        # None: drawn from the OS

    def validate(self) -> None:
        def bad(m):
            raise InvalidArgument("sampling: " + m)
        if not (self.temperature >= 0.0) or self.temperature > 100.0:
            bad("temperature must be in [0, 100]")
        if self.top_k < 0:
            bad("top_k must be >= 0")
        if not (self.top_p > 0.0) or self.top_p > 1.0:
            bad("top_p must be in (0, 1]")
        if not (self.min_p >= 0.0) or self.min_p > 1.0:
            bad("min_p must be in [0, 1]")
        if not (self.repetition_penalty > 0.0):
            bad("repetition_penalty must be > 0")
        if not (abs(self.frequency_penalty) <= 2.0):
            bad("frequency_penalty must be in [-2, 2]")
        if not (abs(self.presence_penalty) <= 2.0):
            bad("presence_penalty must be in [-2, 2]")
        if self.penalty_last_n < -1:
            bad("penalty_last_n must be >= -1")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    @property
    def has_filters(self) -> bool:
        return self.top_k > 1 or self.top_p < 1.0 or self.min_p > 0.0
