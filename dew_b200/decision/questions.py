from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence, Tuple, Union


@dataclass(frozen=True)
class Choice:
    name: str
    options: Tuple[str, ...]


@dataclass(frozen=True)
class Score:
    """A numeric scale answered as a distribution over ``buckets`` equal-width buckets of ``[low, high]``."""
    name: str
    low: float = 0.0
    high: float = 1.0
    buckets: int = 5

    @property
    def options(self) -> Tuple[str, ...]:
        w = (self.high - self.low) / self.buckets
        return tuple(f"{self.low + i * w:g}-{self.low + (i + 1) * w:g}" for i in range(self.buckets))

    def bucket(self, value: float) -> int:
        w = (self.high - self.low) / self.buckets
        return int(min(self.buckets - 1, max(0, (value - self.low) // w)))

    def expectation(self, probs) -> float:
        w = (self.high - self.low) / self.buckets
        return float(sum(p * (self.low + (i + 0.5) * w) for i, p in enumerate(probs)))


Question = Union[Choice, Score]
