"""Frozen-encoder probes: what a representation holds, measured without touching it.  ``features`` runs the encoder over a labelled set
with gradients off and pools its tokens; ``ridge_probe`` fits a linear classifier on them in closed form (ridge regression onto one-hot
targets: one solve, no learning rate, the same answer on every run) and ``knn_probe`` votes among the nearest training features by cosine
similarity with a temperature.  ``ProbeReport`` runs either on a train / validation pair and returns accuracies a validation loop logs.

Reference: src/dew/objectives/jepa/probes.py.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional, Tuple

import torch


@torch.no_grad()
def features(encoder: Callable, batches: Iterable, pool: str = "mean", input_key: str = "image", label_key: str = "label") -> Tuple[torch.Tensor, torch.Tensor]:
    """``(features [N, D], labels [N])``; ``pool``: ``mean`` over tokens, ``first`` (a class token) or ``none`` (the encoder pools)."""
    xs, ys = [], []
    for batch in batches:
        out = encoder(batch[input_key])
        out = out[0] if isinstance(out, tuple) else out
        if out.dim() == 3:
            out = out.mean(1) if pool == "mean" else out[:, 0] if pool == "first" else out.flatten(1)
        xs.append(out.float().cpu())
        ys.append(torch.as_tensor(batch[label_key]).long().cpu())
    return torch.cat(xs), torch.cat(ys)


def _standardise(train: torch.Tensor, *others: torch.Tensor):
    mean, std = train.mean(0, keepdim=True), train.std(0, keepdim=True).clamp_min(1e-6)
    return [(t - mean) / std for t in (train, *others)]


def ridge_probe(train_x, train_y, test_x, test_y, classes: Optional[int] = None, ridge: float = 1e-2) -> Dict[str, float]:
    classes = classes or int(max(train_y.max(), test_y.max())) + 1
    a, b = _standardise(train_x.double(), test_x.double())
    a = torch.cat([a, torch.ones(a.shape[0], 1, dtype=a.dtype)], 1)
    b = torch.cat([b, torch.ones(b.shape[0], 1, dtype=b.dtype)], 1)
    targets = torch.nn.functional.one_hot(train_y, classes).double()
    gram = a.t() @ a + ridge * a.shape[0] * torch.eye(a.shape[1], dtype=a.dtype)
    w = torch.linalg.solve(gram, a.t() @ targets)
    return {"train_accuracy": float(((a @ w).argmax(-1) == train_y).float().mean()), "accuracy": float(((b @ w).argmax(-1) == test_y).float().mean())}


def knn_probe(train_x, train_y, test_x, test_y, k: int = 20, temperature: float = 0.07, classes: Optional[int] = None) -> Dict[str, float]:
    classes = classes or int(max(train_y.max(), test_y.max())) + 1
    a, b = torch.nn.functional.normalize(train_x.float(), dim=-1), torch.nn.functional.normalize(test_x.float(), dim=-1)
    sim, idx = (b @ a.t()).topk(min(k, a.shape[0]), -1)
    votes = torch.zeros(b.shape[0], classes).scatter_add_(1, train_y[idx], (sim / temperature).exp())
    return {"accuracy": float((votes.argmax(-1) == test_y).float().mean())}


class ProbeReport:
    """``ProbeReport(train_batches, val_batches)(encoder) -> {'probe/ridge_accuracy': ..., 'probe/knn_accuracy': ...}``."""

    def __init__(self, train: Iterable, validation: Iterable, pool: str = "mean", input_key: str = "image", label_key: str = "label", k: int = 20,
                 ridge: float = 1e-2):
        self.train, self.validation, self.pool, self.input_key, self.label_key, self.k, self.ridge = list(train), list(validation), pool, input_key, label_key, k, ridge

    def __call__(self, encoder: Callable) -> Dict[str, float]:
        tx, ty = features(encoder, self.train, self.pool, self.input_key, self.label_key)
        vx, vy = features(encoder, self.validation, self.pool, self.input_key, self.label_key)
        r, n = ridge_probe(tx, ty, vx, vy, ridge=self.ridge), knn_probe(tx, ty, vx, vy, self.k)
        return {"probe/ridge_accuracy": r["accuracy"], "probe/ridge_train_accuracy": r["train_accuracy"], "probe/knn_accuracy": n["accuracy"]}
