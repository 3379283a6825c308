"""Few-step generative objectives on the linear (rectified-flow) path ``x_t = (1 - t) x_0 + t eps``, ``v = eps - x_0``.

``MeanFlowObjective``  the network predicts the *average* velocity ``u(x_t, r, t)`` over ``[r, t]``; the MeanFlow identity
                       ``u = v - (t - r) d/dt u`` gives a self-consistent regression target whose total derivative is one
                       Jacobian-vector product (``torch.func.jvp`` with tangents ``(v, 0, 1)``); one step then samples:
                       ``x_0 = x_1 - u(x_1, 0, 1)``.
``ShortcutObjective``  the network takes the step size ``d`` as an input; at ``d = 0`` it regresses the flow-matching velocity,
                       at ``d > 0`` a step of ``2 d`` must equal two of its own steps of ``d`` (targets without gradient).

The model is called as ``model(x, t, r)`` (MeanFlow) or ``model(x, t, d)`` (Shortcut) with ``[rows]`` time tensors.
Reference: src/dew/diffusion/presets.py (``MeanFlow``, ``Shortcut``), src/dew/objectives/diffusion/few_step.py.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import Aux, Objective, Ratio, Step


def _e(t: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    return t.view(-1, *([1] * (x.dim() - 1)))


class MeanFlowObjective(Objective):
    def __init__(self, model, flow_ratio: float = 0.5, adaptive_power: float = 1.0, sample_key: str = "sample", ema_decay: Optional[float] = None):
        self.model, self.flow_ratio, self.p, self.sample_key, self.ema_decay = model, flow_ratio, adaptive_power, sample_key, ema_decay

    def loss(self, variables, batch, step: Step):
        x0 = batch[self.sample_key].float()
        rows = x0.shape[0]
        dev = x0.device
        eps = step.sample("noise", tuple(x0.shape[1:]), rows).to(dev)
        a = step.sample("t", (1,), rows, kind="uniform").to(dev).view(-1)
        b = step.sample("r", (1,), rows, kind="uniform").to(dev).view(-1)
        t, r = torch.maximum(a, b), torch.minimum(a, b)
        same = step.sample("same", (1,), rows, kind="uniform").to(dev).view(-1) < self.flow_ratio
        r = torch.where(same, t, r)                           # a share of pairs is plain flow matching (r = t)
        xt = (1 - _e(t, x0)) * x0 + _e(t, x0) * eps
        v = eps - x0
        fn = lambda x_, r_, t_: self.apply(variables, x_, t_, r_).float()
        u, dudt = torch.func.jvp(fn, (xt, r, t), (v, torch.zeros_like(r), torch.ones_like(t)))
        target = (v - _e(t - r, x0) * dudt).detach()
        err = ((u - target) ** 2).reshape(rows, -1).mean(1)
        weight = 1.0 / (err.detach() + 1e-3) ** self.p        # adaptive loss weight of the MeanFlow recipe
        return Ratio((weight * err).sum(), torch.tensor(float(rows), device=dev)), Aux(metrics={"mse": Ratio(err.detach().sum(), torch.tensor(float(rows), device=dev))})

    @torch.no_grad()
    def generate(self, variables, shape, generator=None, device="cpu", steps: int = 1):
        x = torch.randn(shape, generator=generator).to(device)
        grid = torch.linspace(1.0, 0.0, steps + 1, device=device)
        for i in range(steps):
            t = grid[i].expand(shape[0])
            r = grid[i + 1].expand(shape[0])
            x = x - _e(t - r, x) * self.apply(variables, x, t, r).float()
        return x


class ShortcutObjective(Objective):
    def __init__(self, model, max_log2_steps: int = 7, consistency_share: float = 0.25, sample_key: str = "sample",
                 ema_decay: Optional[float] = None):
        self.model, self.m, self.share, self.sample_key, self.ema_decay = model, max_log2_steps, consistency_share, sample_key, ema_decay

    def loss(self, variables, batch, step: Step):
        x0 = batch[self.sample_key].float()
        rows = x0.shape[0]
        dev = x0.device
        eps = step.sample("noise", tuple(x0.shape[1:]), rows).to(dev)
        k = max(1, int(round(rows * self.share)))             # the first k rows train self-consistency, the rest flow matching
        # flow matching rows: d = 0, any t
        t = step.sample("t", (1,), rows, kind="uniform").to(dev).view(-1)
        d = torch.zeros(rows, device=dev)
        # consistency rows: d = 2^-j for j in 1..m, t on the grid of 2 d so that t - 2 d >= 0
        j = (step.sample("level", (1,), rows, kind="uniform").to(dev).view(-1) * self.m).long().clamp(0, self.m - 1) + 1
        dj = 2.0 ** (-j.float())
        cells = torch.floor(step.sample("cell", (1,), rows, kind="uniform").to(dev).view(-1) / (2 * dj)).clamp_min(1.0)
        tj = (cells * 2 * dj).clamp(max=1.0)
        is_c = torch.arange(rows, device=dev) < k
        t = torch.where(is_c, tj, t)
        d = torch.where(is_c, dj, d)
        xt = (1 - _e(t, x0)) * x0 + _e(t, x0) * eps
        with torch.no_grad():
            tv = step.ema if step.ema is not None else variables
            s1 = self.apply(tv, xt, t, d).float()
            x_mid = xt - _e(d, x0) * s1
            s2 = self.apply(tv, x_mid, t - d, d).float()
            two_steps = 0.5 * (s1 + s2)
        target = torch.where(_e(is_c, x0).bool(), two_steps, eps - x0)
        pred = self.apply(variables, xt, t, torch.where(is_c, 2 * d, d)).float()
        err = ((pred - target) ** 2).reshape(rows, -1).mean(1)
        return Ratio(err.sum(), torch.tensor(float(rows), device=dev)), Aux()

    @torch.no_grad()
    def generate(self, variables, shape, generator=None, device="cpu", steps: int = 1):
        x = torch.randn(shape, generator=generator).to(device)
        d = torch.full((shape[0],), 1.0 / steps, device=device)
        for i in range(steps):
            t = torch.full((shape[0],), 1.0 - i / steps, device=device)
            x = x - _e(d, x) * self.apply(variables, x, t, d).float()
        return x
