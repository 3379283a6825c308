"""Calibration of a classifier's forecasts over K options, and the scores of it: the arithmetic any model's calibration reads.

A forecast is a row of logits (or probabilities) over its real options.  Every function reads held-out forecasts as arrays, so a
model keeps its own policy of which forecasts calibrate together (``dew_b200.decision.calibration`` buckets by question type and
option count).

``fit_temperature``          the temperature minimising the held-out log loss (golden-section search on log T; the loss is unimodal)
``histogram_map`` / ``histogram_mapped``   a top probability -> the held-out accuracy of its bin ``floor(top * bins)``
``abstention_threshold``     the lowest top probability whose accepted forecasts err at most a target, ties counted whole
``reliability_bins`` / ``expected_calibration_error``   per-bin counts (bins closed on the right), additive over passes
``tied_prefixes`` / ``risk_coverage_area``   the area under the risk-coverage curve, equal confidences counted as a whole

Reference: src/dew/eval/calibration.py (the same function names).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np

REJECT_ALL = 1.0 + 1e-9


def softmax(logits, temperature: float = 1.0) -> np.ndarray:
    z = np.asarray(logits, np.float64) / temperature
    z = z - np.max(np.where(np.isfinite(z), z, -np.inf), -1, keepdims=True)
    e = np.where(np.isfinite(z), np.exp(z), 0.0)
    return e / e.sum(-1, keepdims=True)


def _mean_log_loss(logits: np.ndarray, targets: np.ndarray, real: np.ndarray, t: float) -> float:
    z = np.where(real, logits / t, -np.inf)
    z = z - z.max(-1, keepdims=True)
    logp = z - np.log(np.where(real, np.exp(z), 0.0).sum(-1, keepdims=True))
    return float(-(np.where(real & (targets > 0), logp, 0.0) * targets).sum(-1).mean())


def fit_temperature(logits, targets, real=None, lowest: float = 1e-3, highest: float = 100.0) -> float:
    logits, targets = np.asarray(logits, np.float64), np.asarray(targets, np.float64)
    real = np.ones_like(logits, bool) if real is None else np.asarray(real, bool)
    a, b = math.log(lowest), math.log(highest)
    phi = (math.sqrt(5) - 1) / 2
    c, d = b - phi * (b - a), a + phi * (b - a)
    fc, fd = _mean_log_loss(logits, targets, real, math.exp(c)), _mean_log_loss(logits, targets, real, math.exp(d))
    for _ in range(80):
        if fc < fd:
            b, d, fd = d, c, fc
            c = b - phi * (b - a)
            fc = _mean_log_loss(logits, targets, real, math.exp(c))
        else:
            a, c, fc = c, d, fd
            d = a + phi * (b - a)
            fd = _mean_log_loss(logits, targets, real, math.exp(d))
    return float(math.exp((a + b) / 2))


def histogram_map(tops, correct, bins: int = 10) -> np.ndarray:
    """Per bin the held-out accuracy; an empty bin keeps its midpoint."""
    tops, correct = np.asarray(tops, np.float64), np.asarray(correct, np.float64)
    idx = np.clip((tops * bins).astype(int), 0, bins - 1)
    n = np.bincount(idx, minlength=bins).astype(np.float64)
    right = np.bincount(idx, weights=correct, minlength=bins)
    mid = (np.arange(bins) + 0.5) / bins
    return np.where(n > 0, right / np.maximum(n, 1), mid)


def histogram_mapped(top, table: np.ndarray):
    bins = len(table)
    return table[np.clip((np.asarray(top, np.float64) * bins).astype(int), 0, bins - 1)]


def tied_prefixes(confidence, correct) -> List[Tuple[float, int, int]]:
    """Each distinct confidence, highest first, with how many forecasts are at or above it and how many of those are right."""
    conf, right = np.asarray(confidence, np.float64), np.asarray(correct, bool)
    order = np.argsort(-conf, kind="stable")
    conf, right = conf[order], right[order]
    out, i, n, seen_right = [], 0, len(conf), 0
    while i < n:
        j = i
        while j < n and conf[j] == conf[i]:
            j += 1
        seen_right += int(right[i:j].sum())
        out.append((float(conf[i]), j, seen_right))
        i = j
    return out


def abstention_threshold(confidence, correct, target_error: float, conservative: bool = False) -> float:
    best = None
    for c, accepted, right in tied_prefixes(confidence, correct):
        errors = accepted - right
        rate = (errors + 1) / (accepted + 1) if conservative else errors / accepted
        if rate <= target_error:
            best = c
    return REJECT_ALL if best is None else best


def reliability_bins(tops, correct, bins: int = 15) -> np.ndarray:
    """``[3, bins]``: count, summed top probability and number right per bin of (0, 1], closed on the right; passes merge by sum."""
    tops, correct = np.asarray(tops, np.float64), np.asarray(correct, np.float64)
    idx = np.clip(np.ceil(tops * bins).astype(int) - 1, 0, bins - 1)
    return np.stack([np.bincount(idx, minlength=bins).astype(np.float64), np.bincount(idx, weights=tops, minlength=bins),
                     np.bincount(idx, weights=correct, minlength=bins)])


def expected_calibration_error(table: np.ndarray) -> float:
    n, conf, right = table
    total = n.sum()
    return float(np.abs(conf - right).sum() / total) if total else float("nan")


def maximum_calibration_error(table: np.ndarray) -> float:
    n, conf, right = table
    held = n > 0
    return float(np.abs(conf[held] / n[held] - right[held] / n[held]).max()) if held.any() else float("nan")


def risk_coverage_area(confidence, correct) -> float:
    n = len(confidence)
    if n == 0:
        return float("nan")
    area, before = 0.0, 0
    for _, accepted, right in tied_prefixes(confidence, correct):
        area += (accepted - right) / accepted * (accepted - before)
        before = accepted
    return area / n


def brier_score(probabilities, labels) -> float:
    p = np.asarray(probabilities, np.float64)
    onehot = np.eye(p.shape[-1])[np.asarray(labels)]
    return float(((p - onehot) ** 2).sum(-1).mean())
