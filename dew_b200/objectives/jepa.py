"""``JepaObjective``: a context encoder and predictor are trained to predict, in representation space, the output of a
target encoder on masked blocks; the target encoder is the EMA of the context encoder and lives in the trainer's EMA
slot.  Targets are layer-normalised; the loss is L2.

Parity: src/dew/objectives/jepa/objective.py:1-120 (EMA-slot target encoder, LN-normalised targets, L2 loss,
``representation_health`` :66-86), jepa/masking.py (``MultiBlockMask``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..utils import keys as K
from .base import Aux, EMASpec, Moments, Objective, Ratio, Step


@dataclass(frozen=True)
class MultiBlockMask:
    """Sample ``targets`` rectangular target blocks and one context block on a ``grid`` of patches (I-JEPA)."""
    grid: Tuple[int, int] = (14, 14)
    targets: int = 4
    target_scale: Tuple[float, float] = (0.15, 0.2)
    target_aspect: Tuple[float, float] = (0.75, 1.5)
    context_scale: Tuple[float, float] = (0.85, 1.0)

    def _block(self, g: torch.Generator, scale, aspect):
        gh, gw = self.grid
        s = scale[0] + (scale[1] - scale[0]) * float(torch.rand((), generator=g))
        a = aspect[0] + (aspect[1] - aspect[0]) * float(torch.rand((), generator=g))
        area = s * gh * gw
        h = max(1, min(gh, int(round(math.sqrt(area * a)))))
        w = max(1, min(gw, int(round(math.sqrt(area / a)))))
        top = int(torch.randint(0, gh - h + 1, (), generator=g))
        left = int(torch.randint(0, gw - w + 1, (), generator=g))
        m = torch.zeros(gh, gw, dtype=torch.bool)
        m[top:top + h, left:left + w] = True
        return m.reshape(-1)

    def sample(self, key: int):
        """(context mask ``[tokens]``, target mask ``[tokens]``): the context excludes every target block."""
        g = K.generator(key)
        target = torch.zeros(self.grid[0] * self.grid[1], dtype=torch.bool)
        for _ in range(self.targets):
            target |= self._block(g, self.target_scale, self.target_aspect)
        context = self._block(g, self.context_scale, (1.0, 1.0)) & ~target
        if not bool(context.any()):
            context = ~target
        return context, target


def representation_health(z: torch.Tensor) -> dict:
    """Collapse diagnostics of representations ``[B, T, d]``: per-feature std and the effective rank of the batch."""
    flat = z.detach().float().reshape(-1, z.shape[-1])
    std = flat.std(0)
    s = torch.linalg.svdvals(flat - flat.mean(0, keepdim=True))
    p = s / s.sum().clamp_min(1e-12)
    erank = torch.exp(-(p * torch.log(p.clamp_min(1e-12))).sum())
    return {"feature_std": Moments.from_values(std), "effective_rank": Ratio(erank, torch.ones(()))}


class JepaModel(nn.Module):
    """Context encoder + predictor. ``encoder(tokens [B,T,d_in], keep mask) -> [B,T,d]``; the predictor fills mask tokens."""

    def __init__(self, encoder: nn.Module, predictor: nn.Module, features: int):
        super().__init__()
        self.encoder, self.predictor = encoder, predictor
        self.mask_token = nn.Parameter(torch.zeros(features))

    def forward(self, x, context_mask=None):
        z = self.encoder(x)
        if context_mask is None:
            return z
        filled = torch.where(context_mask[None, :, None], z, self.mask_token.to(z.dtype)[None, None])
        return self.predictor(filled)


class JepaObjective(Objective):
    def __init__(self, model: JepaModel, mask: MultiBlockMask = MultiBlockMask(), momentum: float = 0.996, inputs_key: str = "sample"):
        self.model, self.mask, self.inputs_key = model, mask, inputs_key
        self.ema_decay = EMASpec.constant(momentum)           # the EMA slot *is* the target encoder

    def loss(self, variables, batch, step: Step):
        x = batch[self.inputs_key]
        context, target = self.mask.sample(step.fold("mask"))
        context, target = context.to(x.device), target.to(x.device)
        pred = self.apply(variables, x, context)
        with torch.no_grad():
            tgt = self.apply(step.ema if step.ema is not None else variables, x, None)
            tgt = F.layer_norm(tgt.float(), (tgt.shape[-1],))
        err = ((pred.float() - tgt) ** 2).mean(-1)                       # [B, T]
        w = target.float()[None].expand_as(err)
        aux = Aux(metrics=representation_health(tgt))
        return Ratio((err * w).sum(), w.sum()), aux
