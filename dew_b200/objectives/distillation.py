"""``Distillation``: a student matches a frozen teacher's token distribution (forward KL at temperature T), optionally
mixed with the hard-label loss (reference: src/dew/objectives/distillation.py)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .base import Aux, Objective, Ratio, Step


class Distillation(Objective):
    def __init__(self, model, teacher, temperature: float = 1.0, alpha: float = 1.0):
        self.model, self.teacher, self.temperature, self.alpha = model, teacher, temperature, alpha
        for p in self.teacher.parameters():
            p.requires_grad_(False)

    def loss(self, variables, batch, step: Step):
        tokens = batch["tokens"]
        s = self.apply(variables, tokens[:, :-1]).float() / self.temperature
        with torch.no_grad():
            t = self.teacher(tokens[:, :-1]).float() / self.temperature
        kl = (torch.softmax(t, -1) * (torch.log_softmax(t, -1) - torch.log_softmax(s, -1))).sum(-1) * self.temperature ** 2
        per = self.alpha * kl
        if self.alpha < 1.0:
            ce = F.cross_entropy(s.transpose(1, 2) * self.temperature, tokens[:, 1:], reduction="none")
            per = per + (1 - self.alpha) * ce
        n = torch.tensor(float(per.numel()), device=per.device)
        return Ratio(per.sum(), n), Aux(metrics={"teacher_kl": Ratio(kl.detach().sum(), n)})
