from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ..objectives.base import Aux, Objective, Ratio, Step


class DecisionObjective(Objective):
    """Proper scoring rules over the options of every question: ``rule='log'`` (cross-entropy) or ``'brier'``.
    The batch holds ``tokens [B, L]``, ``positions [B, Q]`` and ``answers [B, Q]`` (option index, -1 = unanswered)."""

    def __init__(self, task, rule: str = "log", ema_decay: Optional[float] = None):
        self.model, self.rule, self.ema_decay = task, rule, ema_decay

    def loss(self, variables, batch, step: Step):
        logits = self.model.logits(batch["tokens"], batch["positions"])
        total = torch.zeros((), device=batch["tokens"].device)
        right = torch.zeros((), device=total.device)
        count = torch.zeros((), device=total.device)
        for qi, lg in enumerate(logits):
            y = batch["answers"][:, qi]
            live = y >= 0
            if not bool(live.any()):
                continue
            lg, y = lg[live], y[live]
            if self.rule == "log":
                total = total + F.cross_entropy(lg, y, reduction="sum")
            elif self.rule == "brier":
                total = total + ((torch.softmax(lg, -1) - F.one_hot(y, lg.shape[-1]).float()) ** 2).sum()
            else:
                raise ValueError(f"unknown scoring rule {self.rule!r}; known: log, brier")
            right = right + (lg.argmax(-1) == y).sum()
            count = count + live.sum()
        count = count.clamp_min(1)
        return Ratio(total, count), Aux(metrics={"accuracy": Ratio(right.float(), count)})
