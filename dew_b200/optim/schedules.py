"""Learning-rate schedules as values: ``schedule(step) -> float``.

Parity: src/dew/optim.py (Cosine :1452, Power :1524, Linear / WSD :1609, OneCycle :1668, Exponential :1754).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class Constant:
    value: float

    def __call__(self, step: int) -> float:
        return self.value


@dataclass(frozen=True)
class Cosine:
    peak: float
    steps: int
    warmup: int = 0
    final: float = 0.0
    init: float = 0.0

    def __call__(self, step: int) -> float:
        if self.warmup and step < self.warmup:
            return self.init + (self.peak - self.init) * step / self.warmup
        span = max(1, self.steps - self.warmup)
        u = min(1.0, (step - self.warmup) / span)
        return self.final + 0.5 * (self.peak - self.final) * (1 + math.cos(math.pi * u))


@dataclass(frozen=True)
class Linear:
    """Warm-up, stable plateau, linear decay (WSD when ``decay`` < ``steps``)."""
    peak: float
    steps: int
    warmup: int = 0
    decay: Optional[int] = None
    final: float = 0.0

    def __call__(self, step: int) -> float:
        if self.warmup and step < self.warmup:
            return self.peak * step / self.warmup
        decay = self.steps - self.warmup if self.decay is None else self.decay
        start = self.steps - decay
        if step < start:
            return self.peak
        u = min(1.0, (step - start) / max(1, decay))
        return self.peak + (self.final - self.peak) * u


WSD = Linear


@dataclass(frozen=True)
class Power:
    """``peak * (1 + step / scale)^(-power)`` after warm-up (inverse-sqrt at power 0.5)."""
    peak: float
    power: float = 0.5
    scale: float = 1000.0
    warmup: int = 0

    def __call__(self, step: int) -> float:
        if self.warmup and step < self.warmup:
            return self.peak * step / self.warmup
        return self.peak * (1 + max(0, step - self.warmup) / self.scale) ** (-self.power)


@dataclass(frozen=True)
class OneCycle:
    peak: float
    steps: int
    pct_start: float = 0.3
    div: float = 25.0
    final_div: float = 1e4

    def __call__(self, step: int) -> float:
        up = int(self.steps * self.pct_start)
        lo, end = self.peak / self.div, self.peak / self.final_div
        if step < up:
            return lo + (self.peak - lo) * 0.5 * (1 - math.cos(math.pi * step / max(1, up)))
        u = min(1.0, (step - up) / max(1, self.steps - up))
        return end + (self.peak - end) * 0.5 * (1 + math.cos(math.pi * u))


@dataclass(frozen=True)
class Exponential:
    peak: float
    rate: float = 0.5
    every: int = 1000
    warmup: int = 0
    staircase: bool = False
    final: float = 0.0

    def __call__(self, step: int) -> float:
        if self.warmup and step < self.warmup:
            return self.peak * step / self.warmup
        e = (step - self.warmup) / self.every
        if self.staircase:
            e = math.floor(e)
        return max(self.final, self.peak * self.rate ** e)


def as_schedule(value):
    if callable(value):
        return value
    return Constant(float(value))
