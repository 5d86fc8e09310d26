"""Sampling options with the reference's names, defaults and ranges
(``SamplingConfig``: src/inference.rs:1716-1757; validation :5834-5888)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

from ..errors import SamplingError

_MASK64 = (1 << 64) - 1


@dataclass
class SamplingOptions:
    temperature: float = 0.0            # 0: greedy
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    min_p: Optional[float] = None
    seed: Optional[int] = None          # None: 0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repeat_penalty: float = 1.0
    logit_bias: list = field(default_factory=list)      # (token id, bias) pairs

    def validate(self, vocab_size: int | None = None) -> "SamplingOptions":
        t = self.temperature
        if not isinstance(t, (int, float)) or not math.isfinite(t) or t < 0.0:
            raise SamplingError(f"temperature must be finite and non-negative, got {t}")
        if self.top_k is not None and self.top_k <= 0:
            raise SamplingError("top_k must be greater than zero when provided")
        if self.top_p is not None and not (math.isfinite(self.top_p) and 0.0 < self.top_p <= 1.0):
            raise SamplingError(f"top_p must be finite and in (0, 1], got {self.top_p}")
        if self.min_p is not None and not (math.isfinite(self.min_p) and 0.0 <= self.min_p <= 1.0):
            raise SamplingError(f"min_p must be finite and in [0, 1], got {self.min_p}")
        if not (math.isfinite(self.repeat_penalty) and self.repeat_penalty > 0.0):
            raise SamplingError(f"repeat_penalty must be finite and greater than zero, got {self.repeat_penalty}")
        for name in ("presence_penalty", "frequency_penalty"):
            v = getattr(self, name)
            if not (math.isfinite(v) and -2.0 <= v <= 2.0):
                raise SamplingError(f"{name} must be finite and in [-2, 2], got {v}")
        for tok, bias in self.logit_bias:
            if not (math.isfinite(bias) and -100.0 <= bias <= 100.0):
                raise SamplingError(f"logit_bias for token {tok} must be finite and in [-100, 100], got {bias}")
            if tok < 0 or (vocab_size is not None and tok >= vocab_size):
                raise SamplingError(f"logit_bias token {tok} is outside vocabulary size {vocab_size}")
        if self.seed is not None and not 0 <= self.seed <= _MASK64:
            raise SamplingError(f"seed must fit 64 unsigned bits, got {self.seed}")
        return self

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def adjusts(self) -> bool:
        return (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or self.repeat_penalty != 1.0
                or bool(self.logit_bias))


def splitmix64(state: int) -> int:
    """SplitMix64 finalizer (src/inference.rs:6160-6166)."""
    z = state & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def unit_draw(seed: int, position: int) -> float:
    """Uniform draw in [0, 1) for stream position ``position`` (the length of the history):
    the top 24 bits of splitmix64(seed + (position + 1) * golden) (src/inference.rs:6168-6180).
    It depends on nothing but the seed and the position, so a request draws the same numbers
    alone and inside any batch."""
    state = (seed + (((position + 1) * 0x9E3779B97F4A7C15) & _MASK64)) & _MASK64
    return (splitmix64(state) >> 40) / float(1 << 24)
