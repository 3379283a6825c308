"""The three question types a decision model answers, and the answers it gives.

``Noul``    yes or no (options ``false``, ``true``; the second probability is P(yes))
``Choice``  one of 1..255 named options
``Score``   a rating on 2..10 ordered levels, lowest first; the reported score is the expected level

A question lists its options in a fixed order; the model returns one probability per option in that order.  An answer keeps
that distribution and derives the reported fields (P(yes), the most likely option, the expected level) and a confidence from
it.  ``wire()`` / ``Question.from_wire`` are the JSON request form ``{"type", "instructions", "criteria"}``.

Reference: src/dew/decision/questions.py (Noul / Choice / Score, answers, ``JevConfidence`` / ``TopProbability`` /
``EntropyConfidence``, ``KINDS`` numbering choice 0, score 1, noul 2).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, ClassVar, Dict, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np

JSON = Any


def _need_instructions(instructions: JSON) -> None:
    if instructions is None or (isinstance(instructions, str) and not instructions.strip()):
        raise ValueError("a question needs instructions: what is being asked")


def _distribution(p, n: int) -> np.ndarray:
    p = np.asarray(p, np.float64).reshape(-1)
    if p.shape[0] != n:
        raise ValueError(f"an answer needs one probability per option: {n}, got {p.shape[0]}")
    if not np.all(np.isfinite(p)) or np.any(p < -1e-9):
        raise ValueError("an answer's probabilities are finite and non-negative")
    s = p.sum()
    if not abs(s - 1.0) < 1e-3:
        raise ValueError(f"an answer's probabilities sum to one, got {s:.6f}")
    return np.clip(p, 0.0, None) / s


class Question:
    """One question about a state.  Subclasses define ``kind``, ``options`` and ``descriptions``."""
    kind: ClassVar[str] = ""
    instructions: JSON

    @property
    def options(self) -> Tuple[str, ...]:
        raise NotImplementedError

    @property
    def descriptions(self) -> Tuple[JSON, ...]:
        raise NotImplementedError

    def answer(self, probabilities, confidence: "Confidence" = None, abstained: bool = False):
        raise NotImplementedError

    def wire_criteria(self) -> JSON:
        raise NotImplementedError

    def wire(self) -> Dict[str, JSON]:
        c = self.wire_criteria()
        return {"type": self.kind, "instructions": self.instructions, **({} if c is None else {"criteria": c})}

    @staticmethod
    def from_wire(request: Mapping[str, Any]) -> "Question":
        if not isinstance(request, Mapping):
            raise ValueError(f"a question is a record of type, instructions and criteria, got {type(request).__name__}")
        extra = set(request) - {"type", "instructions", "criteria"}
        if extra:
            raise ValueError(f"a question holds type, instructions and criteria, not {sorted(extra)}")
        kinds = {k.kind: k for k in KINDS}
        kind = request.get("type")
        if kind not in kinds:
            raise ValueError(f"a question's type is one of {sorted(kinds)}, got {kind!r}")
        criteria = request.get("criteria")
        if isinstance(criteria, (bool, int, float, str)):
            raise ValueError(f"a question's criteria are a record, a list or absent, got {criteria!r}")
        return kinds[kind].from_criteria(request.get("instructions"), criteria)

    def index(self, label) -> int:
        """The position of the option ``label`` names (by key, or by integer index)."""
        if isinstance(label, bool) and self.kind == "noul":
            return int(label)
        if isinstance(label, bool) or not isinstance(label, (int, str, np.integer)):
            raise ValueError(f"an answer names an option by key or index, got {label!r}")
        if isinstance(label, (int, np.integer)):
            if not 0 <= int(label) < len(self.options):
                raise ValueError(f"option {label} is outside this question's {len(self.options)} options")
            return int(label)
        if label not in self.options:
            raise ValueError(f"{label!r} is none of this question's options {self.options}")
        return self.options.index(label)


@dataclass(frozen=True)
class Noul(Question):
    instructions: JSON
    criteria: Mapping[str, JSON] = field(default_factory=dict)
    kind: ClassVar[str] = "noul"

    def __post_init__(self):
        _need_instructions(self.instructions)
        extra = set(self.criteria) - {"true", "false"}
        if extra:
            raise ValueError(f"a noul's criteria describe only true and false, got {sorted(extra)}")
        object.__setattr__(self, "criteria", dict(self.criteria))

    def __hash__(self):
        return hash((self.kind, str(self.instructions), tuple(sorted(self.criteria.items(), key=str))))

    @property
    def options(self):
        return ("false", "true")

    @property
    def descriptions(self):
        return (self.criteria.get("false"), self.criteria.get("true"))

    def answer(self, probabilities, confidence=None, abstained=False):
        p = _distribution(probabilities, 2)
        return NoulAnswer(p, (confidence or JevConfidence())(self, p), abstained)

    def wire_criteria(self):
        return dict(self.criteria) or None

    @classmethod
    def from_criteria(cls, instructions, criteria):
        if criteria is not None and not isinstance(criteria, Mapping):
            raise ValueError("a noul's criteria are a record of true / false descriptions")
        return cls(instructions, dict(criteria or {}))


@dataclass(frozen=True)
class Choice(Question):
    instructions: JSON
    criteria: Union[Mapping[str, JSON], Sequence[str]]
    kind: ClassVar[str] = "choice"

    def __post_init__(self):
        _need_instructions(self.instructions)
        c = self.criteria
        if isinstance(c, str) or c is None:
            raise ValueError("a choice's criteria map each option to its description, or list the options")
        pairs = tuple(c.items()) if isinstance(c, Mapping) else tuple((k, None) for k in c)
        if any(not isinstance(k, str) for k, _ in pairs):
            raise ValueError("a choice's options are named by strings")
        if len({k for k, _ in pairs}) != len(pairs):
            raise ValueError("a choice's options must be distinct")
        if not 1 <= len(pairs) <= 255:
            raise ValueError(f"a choice takes 1 to 255 options, got {len(pairs)}")
        object.__setattr__(self, "criteria", dict(pairs))

    def __hash__(self):
        return hash((self.kind, str(self.instructions), tuple(self.criteria)))

    @property
    def options(self):
        return tuple(self.criteria)

    @property
    def descriptions(self):
        return tuple(self.criteria.values())

    def answer(self, probabilities, confidence=None, abstained=False):
        p = _distribution(probabilities, len(self.criteria))
        return ChoiceAnswer(self.options, p, (confidence or JevConfidence())(self, p), abstained)

    def wire_criteria(self):
        return dict(self.criteria)

    @classmethod
    def from_criteria(cls, instructions, criteria):
        if isinstance(criteria, (list, tuple)):
            if any(not isinstance(k, str) for k in criteria):
                raise ValueError("a choice's listed options are strings")
            return cls(instructions, list(criteria))
        if not isinstance(criteria, Mapping):
            raise ValueError("a choice needs criteria: its options")
        return cls(instructions, dict(criteria))

    def restricted(self, options: Sequence[str]) -> "Choice":
        """The same question over ``options`` alone (a tournament round)."""
        return Choice(self.instructions, {o: self.criteria[o] for o in options})


@dataclass(frozen=True)
class Score(Question):
    instructions: JSON
    criteria: Sequence[JSON]
    kind: ClassVar[str] = "score"

    def __post_init__(self):
        _need_instructions(self.instructions)
        if isinstance(self.criteria, (str, Mapping)) or self.criteria is None:
            raise ValueError("a score's criteria list its level descriptions, lowest first")
        levels = tuple(self.criteria)
        if not 2 <= len(levels) <= 10:
            raise ValueError(f"a score takes 2 to 10 levels, got {len(levels)}")
        if any(l is None for l in levels):
            raise ValueError("every score level needs a description")
        object.__setattr__(self, "criteria", levels)

    def __hash__(self):
        return hash((self.kind, str(self.instructions), tuple(str(c) for c in self.criteria)))

    @property
    def options(self):
        return tuple(str(i) for i in range(len(self.criteria)))

    @property
    def descriptions(self):
        return tuple(self.criteria)

    def answer(self, probabilities, confidence=None, abstained=False):
        p = _distribution(probabilities, len(self.criteria))
        return ScoreAnswer(self.descriptions, p, (confidence or JevConfidence())(self, p), abstained)

    def wire_criteria(self):
        return list(self.criteria)

    @classmethod
    def from_criteria(cls, instructions, criteria):
        if not isinstance(criteria, (list, tuple)):
            raise ValueError("a score's criteria list its level descriptions, lowest first")
        return cls(instructions, list(criteria))


# ------------------------------------------------------------------------------------------------ answers
@dataclass(frozen=True)
class NoulAnswer:
    probabilities: np.ndarray
    confidence: float
    abstained: bool = False
    kind: ClassVar[str] = "noul"

    @property
    def noul(self) -> float:
        return float(self.probabilities[1])


@dataclass(frozen=True)
class ChoiceAnswer:
    options: Tuple[str, ...]
    probabilities: np.ndarray
    confidence: float
    abstained: bool = False
    kind: ClassVar[str] = "choice"

    @property
    def choice(self) -> str:
        return self.options[int(np.argmax(self.probabilities))]


@dataclass(frozen=True)
class ScoreAnswer:
    legend: Tuple[JSON, ...]
    probabilities: np.ndarray
    confidence: float
    abstained: bool = False
    kind: ClassVar[str] = "score"

    @property
    def score(self) -> float:
        return float(np.dot(np.arange(len(self.probabilities)), self.probabilities))


Answer = Union[NoulAnswer, ChoiceAnswer, ScoreAnswer]
KINDS: Tuple[type, ...] = (Choice, Score, Noul)     # the numbers a laid-out row gives each type: choice 0, score 1, noul 2


def kind_of(question: Question) -> int:
    return KINDS.index(type(question))


# ------------------------------------------------------------------------------------------------ confidences
class Confidence:
    """A statistic of an answer's distribution, between 0 and 1."""

    def __call__(self, question: Question, probabilities) -> float:
        raise NotImplementedError


class JevConfidence(Confidence):
    """Choice of n options: how far the top probability sits above an even split, ``(p_max - 1/n) / (1 - 1/n)`` (a noul takes
    the same formula over its two options, ``|2p - 1|``; one option is certain).  Score: ``1 - sum_i p_i |i - m| / MAD`` with m
    the most likely level and MAD the mean distance of an even spread from the middle level, floored at 0."""

    def __call__(self, question, probabilities):
        p = np.asarray(probabilities, np.float64)
        n = len(p)
        if isinstance(question, Score):
            peak = int(np.argmax(p))
            levels = np.arange(n)
            spread = float(np.dot(p, np.abs(levels - peak)))
            even = float(np.mean(np.abs(levels - (n - 1) / 2)))
            return min(1.0, max(0.0, 1.0 - spread / even))
        if n == 1:
            return 1.0
        return min(1.0, max(0.0, (float(p.max()) - 1.0 / n) / (1.0 - 1.0 / n)))


class TopProbability(Confidence):
    def __call__(self, question, probabilities):
        return float(np.max(np.asarray(probabilities, np.float64)))


class EntropyConfidence(Confidence):
    """One minus the entropy over the entropy of an even split."""

    def __call__(self, question, probabilities):
        p = np.asarray(probabilities, np.float64)
        if len(p) == 1:
            return 1.0
        h = -float(np.sum(np.where(p > 0, p * np.log(np.clip(p, 1e-300, None)), 0.0)))
        return min(1.0, max(0.0, 1.0 - h / math.log(len(p))))
