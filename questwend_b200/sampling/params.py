"""Sampling options, with the reference's names, meanings and defaults
(``SamplerConfig``, core/sampler.h:16-28; the command line sets the temperature
to 0, cli/main.cpp:134)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8        # <= 0: greedy
    top_p: float = 0.95             # >= 1: off
    top_k: int = 40                 # <= 0: off
    seed: int = 0                   # 0: a fresh random seed
    repeat_penalty: float = 1.0     # logit > 0: divided by it, else multiplied (1: off)
    presence_penalty: float = 0.0   # subtracted once if the token was seen (0: off)
    frequency_penalty: float = 0.0  # subtracted per occurrence (0: off)
    repeat_last_n: int = 64         # the penalty window (<= 0 switches all three off)

    def __post_init__(self):
        if self.temperature > 0 and not self.top_p > 0:
            raise ValueError(f"top_p must be > 0, got {self.top_p}")
        if not self.repeat_penalty > 0:
            raise ValueError(f"repeat_penalty must be > 0, got {self.repeat_penalty}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0

    @property
    def penalized(self) -> bool:
        """core/sampler.cpp:14-18."""
        return self.repeat_last_n > 0 and (self.repeat_penalty != 1.0 or self.presence_penalty != 0.0
                                           or self.frequency_penalty != 0.0)


GREEDY = SamplingParams(temperature=0.0)
