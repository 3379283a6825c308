"""Continual learning measured: a model trained on a sequence of tasks, scored on every task after each.

A run of ``n`` tasks gives an accuracy matrix ``A``, ``A[i][j]`` the accuracy on task ``j``'s test set after training on tasks 0 to ``i``.
Its summaries (Chaudhry et al., arXiv 1801.10112; Lopez-Paz and Ranzato, arXiv 1706.08840): the average accuracy after the last
task; each earlier task's forgetting, the most it lost from its best, ``max_{i < n-1} A[i][j] - A[n-1][j]``; the backward transfer
``mean_j (A[n-1][j] - A[j][j])``, negative where training on later tasks forgot; the forward transfer against a baseline.

Two settings differ in what a task's test chooses among: task-incremental learning scores each example among its own task's classes,
class-incremental learning among every class seen so far.  A language model chooses by the log-likelihood it gives each class's
label after the prompt (``label_scores``).

Reference: src/dew/eval/continual.py (``AccuracyMatrix``, ``continual_run``, ``label_scores``, ``label_accuracy``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class AccuracyMatrix:
    values: np.ndarray            # [stages, tasks], in [0, 1]

    def __post_init__(self):
        v = np.asarray(self.values, np.float64)
        if v.ndim != 2 or v.shape[0] != v.shape[1]:
            raise ValueError("an accuracy matrix has one row a stage and one column a task, as many of each")
        if np.any(v < 0) or np.any(v > 1):
            raise ValueError("accuracies lie in [0, 1]")
        self.values = v

    @property
    def average_accuracy(self) -> float:
        return float(self.values[-1].mean())

    @property
    def forgetting(self) -> np.ndarray:
        """Per earlier task, the most it lost from its best before the last stage."""
        n = len(self.values)
        if n < 2:
            return np.zeros(0)
        return np.array([max(self.values[j:n - 1, j].max() - self.values[-1, j], 0.0) for j in range(n - 1)])

    @property
    def average_forgetting(self) -> float:
        f = self.forgetting
        return float(f.mean()) if len(f) else 0.0

    @property
    def backward_transfer(self) -> float:
        n = len(self.values)
        if n < 2:
            return 0.0
        return float(np.mean([self.values[-1, j] - self.values[j, j] for j in range(n - 1)]))

    def forward_transfer(self, baseline: Sequence[float]) -> float:
        """Mean over tasks j >= 1 of the accuracy on task j just before training on it, less an untrained model's (``baseline[j]``)."""
        n = len(self.values)
        if n < 2:
            return 0.0
        return float(np.mean([self.values[j - 1, j] - baseline[j] for j in range(1, n)]))

    def summary(self) -> dict:
        return {"average_accuracy": self.average_accuracy, "average_forgetting": self.average_forgetting, "backward_transfer": self.backward_transfer}


def continual_run(tasks: Sequence, fit: Callable[[int, object], None], accuracy: Callable[[int, int], float]) -> AccuracyMatrix:
    """Train on ``tasks`` in order and score every task after each: ``fit(i, task)`` trains on task ``i``; ``accuracy(i, j)`` scores
    task ``j`` after it (a class-incremental ``accuracy`` chooses among every class of tasks 0 to ``i``)."""
    n = len(tasks)
    values = np.zeros((n, n))
    for i, task in enumerate(tasks):
        fit(i, task)
        for j in range(n):
            values[i, j] = float(accuracy(i, j))
    return AccuracyMatrix(values)


@torch.no_grad()
def label_scores(model, prompts: Sequence[Sequence[int]], labels: Sequence[Sequence[int]], batch: int = 32, pad_id: int = 0) -> torch.Tensor:
    """``[prompts, labels]``: the log-likelihood the model gives each label's tokens after each prompt."""
    from ..inference.scoring import score
    contexts = [list(p) for p in prompts for _ in labels]
    conts = [list(l) for _ in prompts for l in labels]
    out = score(model, contexts, conts, pad_id=pad_id, batch=batch)
    return torch.tensor([s for s, _, _ in out]).reshape(len(prompts), len(labels))


def label_accuracy(model, prompts, labels, answers: Sequence[int], allowed: Optional[Sequence[int]] = None, **kw) -> float:
    """The share of prompts whose highest-scoring label is their answer; ``allowed`` restricts the choice to those label indices
    (task-incremental scoring: a task's own classes)."""
    s = label_scores(model, prompts, labels, **kw)
    if allowed is not None:
        mask = torch.full((len(labels),), float("-inf"))
        mask[list(allowed)] = 0.0
        s = s + mask
    return float((s.argmax(-1) == torch.tensor(list(answers))).float().mean())
