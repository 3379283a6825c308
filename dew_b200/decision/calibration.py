"""Post-hoc calibration of a decision model: temperatures, binning and abstention, fitted on held-out answers and kept per
bucket (a question type and its option count grouped as 2, 3-5, 6-10, 11+).

``Temperatures``  each question's logits are divided by its bucket's temperature (its type's where the bucket has too few
                  answers), held within ``[lowest, highest]`` - it never sharpens past 0.5
``Binning``       the calibrated top probability is mapped to the accuracy of the held-out answers in its histogram bin
``Abstention``    each bucket's lowest confidence an answer needs: the smallest threshold at or above which the held-out
                  answers err at most a target rate
``Calibration``   the three applied in order: raw logits -> probabilities, reported confidence, abstained or not

Reference: src/dew/decision/calibration.py (``bucket``, ``Scored``, ``Temperatures``, ``Binning``, ``Abstention``, ``Calibration``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np

from .questions import Question


def _count_bucket(n: int) -> str:
    return "2" if n <= 2 else "3-5" if n <= 5 else "6-10" if n <= 10 else "11+"


def bucket(question: Question) -> str:
    return f"{question.kind}:{_count_bucket(len(question.options))}"


@dataclass
class Scored:
    """One held-out answer: the question's type, the raw logits over its options, and the gold distribution over them."""
    kind: str
    logits: np.ndarray
    gold: np.ndarray

    @property
    def bucket(self) -> str:
        return f"{self.kind}:{_count_bucket(len(self.logits))}"

    @classmethod
    def of(cls, question: Question, logits, gold) -> "Scored":
        return cls(question.kind, np.asarray(logits, np.float64), np.asarray(gold, np.float64))


def _softmax(x: np.ndarray) -> np.ndarray:
    z = x - x.max(-1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(-1, keepdims=True)


def _mean_log_loss(group: Sequence[Scored], t: float) -> float:
    total = 0.0
    for s in group:
        z = s.logits / t
        z = z - z.max()
        lp = z - math.log(np.exp(z).sum())
        total -= float(np.dot(s.gold, lp))
    return total / len(group)


def fit_temperature(group: Sequence[Scored], lowest: float = 0.5, highest: float = 10.0) -> float:
    """The temperature in ``[lowest, highest]`` minimising the mean log loss (golden-section search on log T: the loss is
    unimodal in it)."""
    a, b = math.log(lowest), math.log(highest)
    phi = (math.sqrt(5) - 1) / 2
    c, d = b - phi * (b - a), a + phi * (b - a)
    fc, fd = _mean_log_loss(group, math.exp(c)), _mean_log_loss(group, math.exp(d))
    for _ in range(60):
        if fc < fd:
            b, d, fd = d, c, fc
            c = b - phi * (b - a)
            fc = _mean_log_loss(group, math.exp(c))
        else:
            a, c, fc = c, d, fd
            d = a + phi * (b - a)
            fd = _mean_log_loss(group, math.exp(d))
    return float(math.exp((a + b) / 2))


@dataclass
class Temperatures:
    by_bucket: Dict[str, float] = field(default_factory=dict)
    by_kind: Dict[str, float] = field(default_factory=dict)
    lowest: float = 0.5
    highest: float = 10.0

    @classmethod
    def fit(cls, scored: Sequence[Scored], least: int = 20, lowest: float = 0.5, highest: float = 10.0) -> "Temperatures":
        buckets: Dict[str, List[Scored]] = {}
        kinds: Dict[str, List[Scored]] = {}
        for s in scored:
            buckets.setdefault(s.bucket, []).append(s)
            kinds.setdefault(s.kind, []).append(s)
        return cls({b: fit_temperature(g, lowest, highest) for b, g in buckets.items() if len(g) >= least},
                   {k: fit_temperature(g, lowest, highest) for k, g in kinds.items() if len(g) >= 1}, lowest, highest)

    def of(self, kind: str, n: int) -> float:
        t = self.by_bucket.get(f"{kind}:{_count_bucket(n)}", self.by_kind.get(kind, 1.0))
        return min(self.highest, max(self.lowest, t))

    def probabilities(self, kind: str, logits) -> np.ndarray:
        logits = np.asarray(logits, np.float64)
        return _softmax(logits / self.of(kind, logits.shape[-1]))


def _tops(scored: Sequence[Scored], temperatures: Temperatures, binning: Optional["Binning"] = None):
    top, right = [], []
    for s in scored:
        p = temperatures.probabilities(s.kind, s.logits)
        c = float(p.max())
        if binning is not None:
            c = binning.of(s.bucket, c)
        top.append(c)
        right.append(int(np.argmax(p)) == int(np.argmax(s.gold)))
    return np.array(top), np.array(right, bool)


@dataclass
class Binning:
    maps: Dict[str, List[Optional[float]]] = field(default_factory=dict)    # bucket -> per bin accuracy (None: keep the probability)
    bins: int = 10

    @classmethod
    def fit(cls, scored: Sequence[Scored], temperatures: Temperatures, bins: int = 10, least: int = 5) -> "Binning":
        groups: Dict[str, List[Scored]] = {}
        for s in scored:
            groups.setdefault(s.bucket, []).append(s)
        maps = {}
        for b, g in groups.items():
            top, right = _tops(g, temperatures)
            idx = np.clip((top * bins).astype(int), 0, bins - 1)
            row: List[Optional[float]] = []
            for i in range(bins):
                m = idx == i
                row.append(float(right[m].mean()) if m.sum() >= least else None)
            maps[b] = row
        return cls(maps, bins)

    def of(self, bucket_name: str, top: float) -> float:
        row = self.maps.get(bucket_name)
        if row is None:
            return top
        v = row[min(self.bins - 1, max(0, int(top * self.bins)))]
        return top if v is None else v


@dataclass
class Abstention:
    thresholds: Dict[str, float] = field(default_factory=dict)
    default: Optional[float] = None

    @classmethod
    def fit(cls, scored: Sequence[Scored], temperatures: Temperatures, binning: Optional[Binning] = None, target_error: float = 0.05,
            least: int = 20, default: Optional[float] = None) -> "Abstention":
        groups: Dict[str, List[Scored]] = {}
        for s in scored:
            groups.setdefault(s.bucket, []).append(s)
        out = {}
        for b, g in groups.items():
            if len(g) < least:
                continue
            top, right = _tops(g, temperatures, binning)
            order = np.argsort(-top, kind="stable")
            top, wrong = top[order], (~right[order]).astype(float)
            errs = np.cumsum(wrong) / np.arange(1, len(top) + 1)
            # the lowest confidence at which everything at or above it errs at most the target (ties taken whole)
            best = None
            for i in range(len(top)):
                if i + 1 < len(top) and top[i + 1] == top[i]:
                    continue
                if errs[i] <= target_error:
                    best = float(top[i])
            out[b] = best if best is not None else 1.0 + 1e-9        # nothing meets the target: the bucket always abstains
        return cls(out, default)

    def of(self, bucket_name: str) -> Optional[float]:
        return self.thresholds.get(bucket_name, self.default)


@dataclass
class Calibration:
    temperatures: Temperatures = field(default_factory=Temperatures)
    binning: Optional[Binning] = None
    abstention: Optional[Abstention] = None

    @classmethod
    def fit(cls, scored: Sequence[Scored], bins: Optional[int] = 10, target_error: Optional[float] = None, least: int = 20) -> "Calibration":
        t = Temperatures.fit(scored, least)
        b = Binning.fit(scored, t, bins) if bins else None
        a = Abstention.fit(scored, t, b, target_error, least) if target_error is not None else None
        return cls(t, b, a)

    def apply(self, question: Question, logits) -> Tuple[np.ndarray, Optional[float], bool]:
        """``(probabilities, the binned top probability where a map covers it, abstained)``."""
        p = self.temperatures.probabilities(question.kind, logits)
        b = bucket(question)
        top = float(p.max())
        reported = self.binning.of(b, top) if self.binning is not None else top
        gate = self.abstention.of(b) if self.abstention is not None else None
        return p, reported, bool(gate is not None and reported < gate)

    # -- records
    def record(self) -> Dict[str, Any]:
        t = self.temperatures
        return {"temperatures": {"by_bucket": t.by_bucket, "by_kind": t.by_kind, "lowest": t.lowest, "highest": t.highest},
                "binning": None if self.binning is None else {"maps": self.binning.maps, "bins": self.binning.bins},
                "abstention": None if self.abstention is None else {"thresholds": self.abstention.thresholds, "default": self.abstention.default}}

    @classmethod
    def from_record(cls, rec: Mapping[str, Any]) -> "Calibration":
        return cls(Temperatures(**rec["temperatures"]), None if rec.get("binning") is None else Binning(**rec["binning"]),
                   None if rec.get("abstention") is None else Abstention(**rec["abstention"]))
