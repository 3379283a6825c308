"""Guidance wraps a denoiser: CFG, CFG++, APG, Autoguidance (reference: src/dew/sampling/guidance.py:71-506).

A guidance object turns ``(denoiser, unconditional conditions)`` into a callable ``(x, t) -> (x_0, eps)``.
Classifier-free variants evaluate the conditional and unconditional branches as ONE doubled batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

import torch


def _double(conditions: Mapping[str, Any], null: Mapping[str, Any]):
    out = {}
    for k, v in conditions.items():
        n = null.get(k)
        if isinstance(v, torch.Tensor):
            n = torch.zeros_like(v) if n is None else torch.as_tensor(n).to(v).expand_as(v)
            out[k] = torch.cat([v, n], 0)
        else:
            out[k] = v
    return out


class Guidance:
    def wrap(self, denoiser, null_conditions: Optional[Mapping[str, Any]] = None):
        raise NotImplementedError


@dataclass(frozen=True)
class CFG(Guidance):
    """x_0 = x_0^u + scale (x_0^c - x_0^u); optional ``interval=(lo, hi)`` of t/T where guidance applies."""
    scale: float = 3.0
    interval: Optional[tuple] = None

    def combine(self, cond, uncond, x, t, denoiser):
        return uncond + self.scale * (cond - uncond)

    def wrap(self, denoiser, null_conditions=None):
        null = dict(null_conditions or {})
        doubled = _double(denoiser.conditions, null)

        def guided(x, t):
            t = torch.as_tensor(t, device=x.device, dtype=torch.float32)
            tt = t.expand(x.shape[0]) if t.dim() == 0 else t
            if self.scale == 1.0 or not denoiser.conditions:
                return denoiser(x, tt)
            raw = denoiser.raw(torch.cat([x, x], 0), torch.cat([tt, tt], 0), doubled)
            x0, _ = denoiser.convert(torch.cat([x, x], 0), torch.cat([tt, tt], 0), raw)
            c, u = x0.chunk(2, 0)
            g = self.combine(c, u, x, tt, denoiser)
            if self.interval is not None:
                T = denoiser.schedule.T
                inside = ((tt / T >= self.interval[0]) & (tt / T <= self.interval[1])).reshape(-1, *([1] * (x.dim() - 1)))
                g = torch.where(inside, g, c)
            a, s = denoiser.process.rates(tt, like=x) if denoiser.schedule is denoiser.process.sampler_schedule() else \
                __import__("dew_b200.diffusion.transforms", fromlist=["broadcast_rates"]).broadcast_rates(denoiser.schedule, tt, x)
            eps = (x - a * g) / s.clamp_min(1e-20)
            if isinstance(self, CFGPlusPlus):  # renoise with the unconditional eps
                eps = (x - a * u) / s.clamp_min(1e-20)
            return g, eps
        return guided


@dataclass(frozen=True)
class CFGPlusPlus(CFG):
    """CFG++ (Chung et al. 2024): guided clean estimate, unconditional noise for the re-noising step."""
    scale: float = 0.6

    def combine(self, cond, uncond, x, t, denoiser):
        return uncond + self.scale * (cond - uncond)


@dataclass(frozen=True)
class APG(CFG):
    """Adaptive projected guidance: down-weight the update's component parallel to the conditional prediction,
    rescale its norm to ``norm_threshold`` and keep a negative-momentum running average (Sadat et al. 2024)."""
    scale: float = 7.5
    eta: float = 0.0
    norm_threshold: float = 0.0
    momentum: float = 0.0

    def combine(self, cond, uncond, x, t, denoiser):
        diff = cond - uncond
        dims = tuple(range(1, diff.dim()))
        if self.norm_threshold > 0:
            n = diff.norm(dim=dims, keepdim=True)
            diff = diff * torch.minimum(torch.ones_like(n), self.norm_threshold / n.clamp_min(1e-12))
        unit = cond / cond.norm(dim=dims, keepdim=True).clamp_min(1e-12)
        par = (diff * unit).sum(dim=dims, keepdim=True) * unit
        orth = diff - par
        return cond + (self.scale - 1) * (orth + self.eta * par)


@dataclass(frozen=True)
class Autoguidance(Guidance):
    """Guide a model with a weaker version of itself (Karras et al. 2024): D = D_weak + scale (D - D_weak)."""
    weak: Any = None
    scale: float = 2.0

    def wrap(self, denoiser, null_conditions=None):
        def guided(x, t):
            x0, _ = denoiser(x, t)
            w0, _ = self.weak(x, t)
            g = w0 + self.scale * (x0 - w0)
            tt = torch.as_tensor(t, device=x.device, dtype=torch.float32)
            tt = tt.expand(x.shape[0]) if tt.dim() == 0 else tt
            from ..diffusion.transforms import broadcast_rates
            a, s = broadcast_rates(denoiser.schedule, tt, x)
            return g, (x - a * g) / s.clamp_min(1e-20)
        return guided
