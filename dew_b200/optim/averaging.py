"""Weight averaging: ``ema_update`` (``decay * avg + (1 - decay) * live`` in >= fp32), EDM2 power-function
profiles and post-hoc EMA coefficients.

Parity: src/dew/averaging.py:116-139 (``ema_update``), ``power_decay``, post-hoc ``coefficients``.
"""
from __future__ import annotations

import math
from typing import Any, Mapping, Sequence

import numpy as np
import torch

from .. import ops
from ..utils.trees import tree_map


def ema_update(avg: Any, live: Any, decay: float) -> Any:
    """In-place leaf-wise EMA; integer / bool leaves and leaves that are the same object are left as they are."""
    def one(a, l):
        if not isinstance(a, torch.Tensor) or not a.dtype.is_floating_point or a is l:
            return a
        ops.ema_(a, l.detach(), decay)
        return a
    with torch.no_grad():
        return tree_map(one, avg, live)


def gamma_of_std(std: float) -> float:
    """Solve the EDM2 relation between a power profile's exponent gamma and its relative standard deviation."""
    tmp = std ** -2
    r = np.roots([1, 7, 16 - tmp, 12 - tmp]).real.max()
    return float(r)


def power_decay(step: int, gamma: float) -> float:
    return (1 - 1 / max(step, 1)) ** (gamma + 1)


def _dot(ta, ga, tb, gb):
    """Inner product of two power profiles p(t) ~ t^gamma on [0, t_a] and [0, t_b] (Karras et al. 2024, Alg. 2)."""
    tmax = np.maximum(ta, tb)
    tmin = np.minimum(ta, tb)
    ratio = tmin / tmax
    g = np.where(ta > tb, gb, ga)   # exponent of the shorter profile inside the integral
    num = (ga + 1) * (gb + 1) * ratio ** g
    den = (ga + gb + 1) * tmax
    return num / den


def coefficients(steps: Sequence[int], gammas: Sequence[float], target_step: int, target_gamma: float) -> np.ndarray:
    """Least-squares weights over stored snapshots (step_i, gamma_i) reproducing a target power profile."""
    t = np.asarray(steps, dtype=np.float64)
    g = np.asarray(gammas, dtype=np.float64)
    A = _dot(t[:, None], g[:, None], t[None, :], g[None, :])
    b = _dot(t, g, np.float64(target_step), np.float64(target_gamma))
    return np.linalg.lstsq(A, b, rcond=None)[0]


def posthoc_average(snapshots: Sequence[Mapping[str, Any]], weights: Sequence[float]) -> Any:
    out = tree_map(lambda x: x.float() * float(weights[0]) if isinstance(x, torch.Tensor) else x, snapshots[0])
    for snap, w in zip(snapshots[1:], weights[1:]):
        out = tree_map(lambda a, b: a + b.float() * float(w) if isinstance(a, torch.Tensor) else a, out, snap)
    return out
