"""Proper scoring rules: the losses a decision model trains on and the scores it is judged by.

A rule charges a forecast ``p = softmax(logits over the row's real options)`` for a target distribution ``t`` (one-hot or soft);
a proper rule charges least in expectation when ``p`` is the true distribution.  ``charge(logits, target, options, ordinal)``
takes ``[R, K]`` logits (anything past a row's options), ``[R, K]`` targets, the ``[R, K]`` mask of real options and the ``[R]``
flag of rows whose options are ordered levels, and returns ``[R]`` charges, zero for a certain and correct forecast.  Rules add
and scale: ``LogLoss() + 0.5 * Brier()``.

Reference: src/dew/decision/scoring.py (``LogLoss``, ``Brier``, ``Spherical``, ``RankedProbability``, ``Combined``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch


def masked_log_softmax(logits: torch.Tensor, options: torch.Tensor) -> torch.Tensor:
    x = (logits if logits.dtype == torch.float64 else logits.float()).masked_fill(~options, float("-inf"))
    # a row without any option (padding) would give NaN: give it one fake option
    empty = ~options.any(-1, keepdim=True)
    x = torch.where(empty, torch.zeros_like(x), x)
    return torch.log_softmax(x, -1)


def probabilities(logits: torch.Tensor, options: torch.Tensor) -> torch.Tensor:
    return masked_log_softmax(logits, options).exp() * options


class ScoringRule:
    name = "rule"
    lower_is_better = True

    def charge(self, logits, target, options, ordinal) -> torch.Tensor:
        raise NotImplementedError

    def __add__(self, other: "ScoringRule") -> "Combined":
        return Combined(((1.0, self),)) + other

    def __mul__(self, w: float) -> "Combined":
        return Combined(((float(w), self),))

    __rmul__ = __mul__

    # as a metric over a ``Decisions`` artifact: (total, count)
    def __call__(self, decisions) -> Tuple[float, float]:
        scored = decisions.scored
        if not bool(scored.any()):
            return 0.0, 0.0
        logits = decisions.probabilities.double().clamp_min(1e-300).log()
        c = self.charge(logits[scored], decisions.targets[scored].double(), decisions.options[scored], decisions.ordinal[scored])
        return float(c.sum()), float(scored.sum())


@dataclass(frozen=True)
class LogLoss(ScoringRule):
    """The cross entropy ``-sum_k t_k log p_k``: a one-hot target is charged ``-log p_y``."""
    name = "log_loss"

    def charge(self, logits, target, options, ordinal):
        lp = masked_log_softmax(logits, options)
        return -(torch.where(options & (target > 0), lp, torch.zeros_like(lp)) * target).sum(-1)


@dataclass(frozen=True)
class Brier(ScoringRule):
    """``sum_k (p_k - t_k)^2``, between 0 and 2."""
    name = "brier"

    def charge(self, logits, target, options, ordinal):
        p = probabilities(logits, options)
        return ((p - target * options) ** 2).sum(-1)


@dataclass(frozen=True)
class Spherical(ScoringRule):
    """``1 - (t . p) / |p|``, between 0 and 1."""
    name = "spherical"

    def charge(self, logits, target, options, ordinal):
        p = probabilities(logits, options)
        return 1.0 - (p * target).sum(-1) / p.norm(dim=-1).clamp_min(1e-12)


@dataclass(frozen=True)
class RankedProbability(ScoringRule):
    """Ordered levels only: the squared gaps between the cumulative forecast and the cumulative target over the K - 1 cuts,
    ``sum_k (P_k - T_k)^2 / (K - 1)``; rows whose options have no order are charged nothing."""
    name = "rps"

    def charge(self, logits, target, options, ordinal):
        p = probabilities(logits, options)
        gaps = (p.cumsum(-1) - (target * options).cumsum(-1)) ** 2
        k = options.sum(-1)
        cuts = options & (torch.arange(options.shape[-1], device=options.device)[None] < (k[:, None] - 1))
        c = (gaps * cuts).sum(-1) / (k - 1).clamp_min(1)
        return torch.where(ordinal, c, torch.zeros_like(c))

    def __call__(self, decisions):
        total, _ = super().__call__(decisions)
        return total, float((decisions.scored & decisions.ordinal).sum())


@dataclass(frozen=True)
class Combined(ScoringRule):
    terms: Tuple[Tuple[float, ScoringRule], ...]

    def __post_init__(self):
        if any(w <= 0 for w, _ in self.terms):
            raise ValueError("a sum of proper scoring rules stays proper only with positive weights")

    @property
    def name(self):
        return "+".join(r.name if w == 1 else f"{w:g}*{r.name}" for w, r in self.terms)

    def charge(self, logits, target, options, ordinal):
        out = None
        for w, r in self.terms:
            c = w * r.charge(logits, target, options, ordinal)
            out = c if out is None else out + c
        return out

    def __add__(self, other):
        return Combined(self.terms + (other.terms if isinstance(other, Combined) else ((1.0, other),)))

    def __mul__(self, w):
        return Combined(tuple((float(w) * h, r) for h, r in self.terms))

    __rmul__ = __mul__


def rule_named(name: str) -> ScoringRule:
    table = {"log": LogLoss(), "log_loss": LogLoss(), "brier": Brier(), "spherical": Spherical(), "rps": RankedProbability()}
    if name not in table:
        raise ValueError(f"unknown scoring rule {name!r}; known: {sorted(table)}")
    return table[name]
