"""Sampling parameters with the reference's names, defaults and checks
(crates/core/src/lib.rs:23-65)."""
from __future__ import annotations

import math
from dataclasses import dataclass

from ..errors import InvalidRequest


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int | None = None
    top_p: float = 1.0
    seed: int = 0
    max_tokens: int = 128
    ignore_eos: bool = False

    def validate(self) -> None:
        if not isinstance(self.temperature, (int, float)) or not math.isfinite(self.temperature) or self.temperature < 0:
            raise InvalidRequest("temperature must be finite and nonnegative")
        if not isinstance(self.top_p, (int, float)) or not math.isfinite(self.top_p) or not 0.0 < self.top_p <= 1.0:
            raise InvalidRequest("top_p must be in (0, 1]")
        if (self.top_k is not None and (not isinstance(self.top_k, int) or self.top_k <= 0)) \
                or not isinstance(self.max_tokens, int) or self.max_tokens <= 0:
            raise InvalidRequest("top_k and max_tokens must be positive")
        if not isinstance(self.seed, int) or not 0 <= self.seed < 2**64:
            raise InvalidRequest("seed must be an unsigned 64-bit integer")

    def is_greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1
