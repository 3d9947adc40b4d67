"""Sampling and generation options, with the reference's names, defaults and checks."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

from ..errors import OptionsError


@dataclass
class Sampling:
    """crates/llama-rs/src/sampling.rs:3-36: temperature 0 is greedy; top_k 0 is off."""

    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    seed: int = 42

    def validate(self) -> None:
        ok = (math.isfinite(self.temperature) and self.temperature >= 0.0
              and math.isfinite(self.top_p) and 0.0 < self.top_p <= 1.0
              and math.isfinite(self.repeat_penalty) and self.repeat_penalty > 0.0
              and self.top_k >= 0 and self.repeat_last_n >= 0)
        if not ok:
            raise OptionsError("invalid sampling parameters")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 and self.repeat_penalty == 1.0

    @property
    def plain_temperature(self) -> bool:
        """Temperature alone: no top-k, no top-p cut, no penalty."""
        return (self.temperature > 0.0 and self.top_k == 0 and self.top_p >= 1.0
                and self.repeat_penalty == 1.0)


@dataclass
class GenerationOptions:
    """crates/llama-rs/src/lib.rs:98-110."""

    max_tokens: int = 256
    sampling: Sampling = field(default_factory=Sampling)

    def validate(self) -> None:
        self.sampling.validate()
        if self.max_tokens <= 0:
            raise OptionsError("max_tokens must be positive")
