"""``DPO``: direct preference optimisation with the frozen reference policy held in the trainer's EMA slot (decay 1),
as the reference's demo does (examples/readme_demo.py:105-138; src/dew/objectives/rl DPO)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ..base import Aux, EMASpec, Objective, Ratio, Step


def sequence_logprob(logits: torch.Tensor, tokens: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Sum over scored positions of log p(token_t | tokens_<t); ``logits [B,S-1,V]`` predict ``tokens[:, 1:]``."""
    lp = torch.log_softmax(logits.float(), -1).gather(-1, tokens[:, 1:, None]).squeeze(-1)
    return (lp * mask[:, 1:].float()).sum(-1)


class DPO(Objective):
    starts_from_model = True
    def __init__(self, model, beta: float = 0.1, label_smoothing: float = 0.0):
        self.model, self.beta, self.label_smoothing = model, beta, label_smoothing
        self.ema_decay = EMASpec.constant(1.0)          # the EMA slot never moves: it is the reference policy

    def _lp(self, variables, tokens, mask):
        return sequence_logprob(self.apply(variables, tokens[:, :-1]), tokens, mask)

    def loss(self, variables, batch, step: Step):
        pc, pr = self._lp(variables, batch["chosen"], batch["chosen_mask"]), self._lp(variables, batch["rejected"], batch["rejected_mask"])
        with torch.no_grad():
            ref = step.ema if step.ema is not None else variables
            rc, rr = self._lp(ref, batch["chosen"], batch["chosen_mask"]), self._lp(ref, batch["rejected"], batch["rejected_mask"])
        margin = self.beta * ((pc - rc) - (pr - rr))
        per = -(1 - self.label_smoothing) * F.logsigmoid(margin) - self.label_smoothing * F.logsigmoid(-margin)
        n = torch.tensor(float(per.shape[0]), device=per.device)
        aux = Aux(metrics={"reward_accuracy": Ratio((margin > 0).float().sum(), n), "reward_margin": Ratio(margin.detach().sum(), n)})
        return Ratio(per.sum(), n), aux
