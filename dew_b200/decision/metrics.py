"""Metrics of a decision model's answers over a validation pass.

Each metric reads ``Decisions`` (one row per asked question: the model's probabilities over its options, the gold distribution,
which rows have a known answer) and returns partial totals that ``merge`` adds over batches and ``finalize`` turns into the
number, so a split's metric does not depend on how it was batched.  The proper scoring rules are metrics too
(``scoring.ScoringRule.__call__``).

Reference: src/dew/decision/metrics.py (``Accuracy``, ``MacroF1``, ``ECE`` with 15 bins closed on the right, ``AURC``,
``ScoredQuestions``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Sequence, Tuple

import numpy as np
import torch


@dataclass
class Decisions:
    probabilities: torch.Tensor    # [M, K]
    targets: torch.Tensor          # [M, K]
    options: torch.Tensor          # [M, K] bool
    scored: torch.Tensor           # [M] bool: has a known answer
    ordinal: torch.Tensor          # [M] bool: a score question
    classes: torch.Tensor          # [M] int64: an id of the question asked (equal questions share it)

    @staticmethod
    def cat(parts: Sequence["Decisions"]) -> "Decisions":
        K = max(p.probabilities.shape[1] for p in parts)
        def pad(x):
            return torch.nn.functional.pad(x, (0, K - x.shape[1]))
        return Decisions(torch.cat([pad(p.probabilities) for p in parts]), torch.cat([pad(p.targets) for p in parts]),
                         torch.cat([pad(p.options) for p in parts]), torch.cat([p.scored for p in parts]),
                         torch.cat([p.ordinal for p in parts]), torch.cat([p.classes for p in parts]))

    def tops(self) -> Tuple[np.ndarray, np.ndarray]:
        """Each answered question's top probability and whether its top option is the right one."""
        s = self.scored
        p = self.probabilities[s].double()
        top, idx = p.max(-1)
        right = idx == self.targets[s].argmax(-1)
        return top.cpu().numpy(), right.cpu().numpy()


class Metric:
    name = "metric"
    lower_is_better = False

    def __call__(self, d: Decisions):
        raise NotImplementedError

    @staticmethod
    def merge(a, b):
        return tuple(x + y for x, y in zip(a, b))

    @staticmethod
    def finalize(t) -> float:
        return float(t[0] / t[1]) if t[1] else float("nan")


class Accuracy(Metric):
    name = "accuracy"

    def __call__(self, d):
        _, right = d.tops()
        return float(right.sum()), float(len(right))


class ScoredQuestions(Metric):
    name = "scored_questions"

    def __call__(self, d):
        return float(d.scored.sum()), 1.0

    @staticmethod
    def merge(a, b):
        return (a[0] + b[0], 1.0)


class MacroF1(Metric):
    """The mean over classes of each class's F1; a class is (question, option).  True / false positives and false negatives add
    over the whole pass before any F1 is taken."""
    name = "macro_f1"

    def __call__(self, d):
        s = d.scored
        pred = d.probabilities[s].argmax(-1)
        gold = d.targets[s].argmax(-1)
        base = d.classes[s] * 256
        counts: Dict[int, List[int]] = {}
        for p, g, b in zip(pred.tolist(), gold.tolist(), base.tolist()):
            if p == g:
                counts.setdefault(b + g, [0, 0, 0])[0] += 1
            else:
                counts.setdefault(b + p, [0, 0, 0])[1] += 1
                counts.setdefault(b + g, [0, 0, 0])[2] += 1
        return (counts,)

    @staticmethod
    def merge(a, b):
        out = {k: list(v) for k, v in a[0].items()}
        for k, v in b[0].items():
            cur = out.setdefault(k, [0, 0, 0])
            for i in range(3):
                cur[i] += v[i]
        return (out,)

    @staticmethod
    def finalize(t):
        f1 = [2 * tp / (2 * tp + fp + fn) if (2 * tp + fp + fn) else 0.0 for tp, fp, fn in t[0].values()]
        return float(np.mean(f1)) if f1 else float("nan")


class ECE(Metric):
    """Expected calibration error over ``bins`` equal bins on (0, 1], closed on the right, weighted by their counts."""
    name = "ece"
    lower_is_better = True

    def __init__(self, bins: int = 15):
        self.bins = bins

    def __call__(self, d):
        top, right = d.tops()
        idx = np.clip(np.ceil(top * self.bins).astype(int) - 1, 0, self.bins - 1)
        conf = np.bincount(idx, weights=top, minlength=self.bins)
        acc = np.bincount(idx, weights=right.astype(float), minlength=self.bins)
        n = np.bincount(idx, minlength=self.bins).astype(float)
        return conf, acc, n

    @staticmethod
    def finalize(t):
        conf, acc, n = t
        total = n.sum()
        return float(np.abs(conf - acc).sum() / total) if total else float("nan")


class AURC(Metric):
    """Area under the risk-coverage curve: the error rate among the rows at or above each confidence, weighted by how many rows
    that confidence adds (equal confidences count as a whole, in any row order).  Lower is better."""
    name = "aurc"
    lower_is_better = True

    def __call__(self, d):
        top, right = d.tops()
        return (list(zip(top.tolist(), right.tolist())),)

    @staticmethod
    def merge(a, b):
        return (a[0] + b[0],)

    @staticmethod
    def finalize(t):
        rows = t[0]
        if not rows:
            return float("nan")
        conf = np.array([c for c, _ in rows])
        wrong = 1.0 - np.array([float(r) for _, r in rows])
        order = np.argsort(-conf, kind="stable")
        conf, wrong = conf[order], wrong[order]
        n = len(rows)
        area, seen, errors, i = 0.0, 0, 0.0, 0
        while i < n:
            j = i
            while j < n and conf[j] == conf[i]:
                j += 1
            errors += wrong[i:j].sum()
            seen = j
            area += (errors / seen) * (j - i)
            i = j
        return float(area / n)


def default_metrics() -> List[Any]:
    """Accuracy, macro F1, calibration error, risk-coverage area, log loss, Brier score and the count they are taken over."""
    from .scoring import Brier, LogLoss
    return [Accuracy(), MacroF1(), ECE(), AURC(), _RuleMetric(LogLoss()), _RuleMetric(Brier()), ScoredQuestions()]


class _RuleMetric(Metric):
    lower_is_better = True

    def __init__(self, rule):
        self.rule, self.name = rule, rule.name

    def __call__(self, d):
        return self.rule(d)


def measure(batches: Sequence[Decisions], metrics=None) -> Dict[str, float]:
    metrics = metrics if metrics is not None else default_metrics()
    out = {}
    for m in metrics:
        total = None
        for d in batches:
            part = m(d)
            total = part if total is None else m.merge(total, part)
        out[m.name] = m.finalize(total) if total is not None else float("nan")
    return out
