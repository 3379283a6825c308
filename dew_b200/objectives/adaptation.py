"""Test-time training over the task loss: a continuum level stepped in context, a window at a time.

Nested Learning's continuum memory (Behrouz et al., arXiv 2512.24695, section 7.1, eq. 71) steps a block's parameters every
``C`` tokens by the gradient of the model's own objective over them: ``theta <- theta - eta * sum_{t in window} grad L(theta;
x_t)`` at each window's end, the window's tokens read at the theta it opened with.  The level is a residual two-layer map
``x + U act(D x)`` on the decoder's final states before its head (``U`` starts at zero, so the model gains the level as the
identity).  The trunk runs once; each window's states go through the level at that window's parameters and the model's own
head; the next-token losses there are the objective's, and their gradient steps the level for the next window.  The outer
loss differentiates through every step (the second-order meta-gradient of the level's start), or not (``first_order``).
Each row adapts by itself: the level's parameters carry a leading row axis inside the loop.

Reference: src/dew/nn/continuum.py (``Continuum``), src/dew/objectives/lm/adaptation.py (``ChunkAdaptation``, the windowed scan).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .base import Aux, Exponentiated, Objective, Ratio, Step


class Continuum(nn.Module):
    """``x + U act(D x)``; ``U`` starts at zero."""

    def __init__(self, features: int, hidden: int):
        super().__init__()
        self.down = nn.Parameter(torch.randn(hidden, features) / features ** 0.5)
        self.up = nn.Parameter(torch.zeros(features, hidden))

    def forward(self, x):
        return x + F.linear(F.silu(F.linear(x, self.down)), self.up)

    @staticmethod
    def apply_rows(params: Dict[str, torch.Tensor], x: torch.Tensor) -> torch.Tensor:
        """One level per row: ``params`` carry a leading row axis ``[B, ...]``, ``x [B, C, d]``."""
        h = F.silu(torch.einsum("bcd,bhd->bch", x, params["down"]))
        return x + torch.einsum("bch,bdh->bcd", h, params["up"])


@dataclass(frozen=True)
class ChunkAdaptation:
    window: int = 64            # C: tokens per step of the level
    rate: float = 1e-2          # eta
    first_order: bool = False   # drop the meta-gradient through the steps (cheaper, biased)

    def __post_init__(self):
        if self.window < 1 or not self.rate > 0:
            raise ValueError("an adaptation steps every window >= 1 tokens at a positive rate")


class _WithLevel(nn.Module):
    def __init__(self, backbone: nn.Module, level: Continuum):
        super().__init__()
        self.backbone, self.continuum = backbone, level

    def forward(self, *args, **kwargs):
        return self.backbone(*args, **kwargs)


class AdaptiveLMObjective(Objective):
    """Next-token loss of a decoder whose final states pass through a continuum level that is stepped in context.
    ``model`` needs ``forward(tokens, return_hidden=True)`` and ``logits(hidden)`` (``CausalTransformer`` has both)."""

    def __init__(self, model: nn.Module, seq_len: int, adaptation: ChunkAdaptation = ChunkAdaptation(), level_features: int = None,
                 level_hidden: int = None, ema_decay=None):
        d = level_features or model.config.emb_features
        level = Continuum(d, level_hidden or d)
        p = next(model.parameters(), None)
        if p is not None:
            level = level.to(p.device)
        self.model = _WithLevel(model, level)
        self.seq_len, self.adaptation, self.ema_decay = seq_len, adaptation, ema_decay

    def _window_losses(self, hidden, targets, start: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        """(per-token losses ``[B, S]`` with the level stepped window by window, norm of the level's last step per row)."""
        B, S, _ = hidden.shape
        C, eta = self.adaptation.window, self.adaptation.rate
        theta = {k: v[None].expand(B, *v.shape) for k, v in start.items()}           # every row starts from the trained start
        if not any(v.requires_grad for v in theta.values()):
            theta = {k: v.detach().requires_grad_() for k, v in theta.items()}
        out = []
        moved = torch.zeros(B, device=hidden.device)
        for lo in range(0, S, C):
            states = Continuum.apply_rows(theta, hidden[:, lo:lo + C])
            logits = self.model.backbone.logits(states).float()
            tl = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets[:, lo:lo + C].reshape(-1), reduction="none", ignore_index=-100)
            tl = tl.view(B, -1)
            out.append(tl)
            if lo + C < S:
                grads = torch.autograd.grad(tl.sum(), list(theta.values()), create_graph=not self.adaptation.first_order, retain_graph=True, allow_unused=True)
                new = {}
                for (k, v), g in zip(theta.items(), grads):
                    g = torch.zeros_like(v) if g is None else (g.detach() if self.adaptation.first_order else g)
                    new[k] = v - eta * g
                moved = sum((new[k] - theta[k]).detach().reshape(B, -1).pow(2).sum(1) for k in theta).sqrt()
                theta = new
        return torch.cat(out, 1), moved

    def loss(self, variables, batch, step: Step):
        tokens = batch["tokens"]
        inputs, targets = tokens[:, :-1], tokens[:, 1:].clone()
        if "loss_mask" in batch:
            targets[batch["loss_mask"][:, 1:] == 0] = -100
        with torch.enable_grad():
            hidden = self.apply(variables, inputs, return_hidden=True)
            if variables is not None:
                from ..utils.trees import variables_for_call
                flat = variables_for_call(self.model, variables)
                start = {"down": flat["continuum.down"], "up": flat["continuum.up"]}
            else:
                start = {"down": self.model.continuum.down, "up": self.model.continuum.up}
            per_token, moved = self._window_losses(hidden, targets, start)
        scored = (targets != -100).float()
        mass = scored.sum()
        total = (per_token * scored).sum()
        if not step.train:
            total = total.detach()
        return Ratio(total, mass), Aux(metrics={"perplexity": Exponentiated(Ratio(total.detach(), mass)),
                                                "level_step": Ratio(moved.sum(), torch.tensor(float(moved.shape[0]), device=moved.device))})
