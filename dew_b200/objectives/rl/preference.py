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
    def __init__(self, model, beta: float = 0.1, label_smoothing: float = 0.0, share_prefix: bool = False, min_prefix: int = 8):
        """``share_prefix``: a pair's two halves begin with the same prompt; lay it out once per pair (``data.forked_rows``) instead of
        once per half - the same loss and gradients for about the prompt's share fewer tokens."""
        self.model, self.beta, self.label_smoothing = model, beta, label_smoothing
        self.share_prefix, self.min_prefix = share_prefix, min_prefix
        self.ema_decay = EMASpec.constant(1.0)          # the EMA slot never moves: it is the reference policy

    def _lp(self, variables, tokens, mask):
        return sequence_logprob(self.apply(variables, tokens[:, :-1]), tokens, mask)

    def _pair_lp(self, variables, batch):
        """Both halves through one forked layout: ``(chosen log-probabilities, rejected log-probabilities)``."""
        from .policy import forked_logits
        c, r = batch["chosen"], batch["rejected"]
        S = max(c.shape[1], r.shape[1])
        pad = lambda t: F.pad(t, (0, S - t.shape[1]))
        tokens = torch.stack([pad(c), pad(r)], 1).reshape(-1, S)                      # chosen_0, rejected_0, chosen_1, ...
        mask = torch.stack([pad(batch["chosen_mask"]), pad(batch["rejected_mask"])], 1).reshape(-1, S)
        logits = forked_logits(lambda *a, **k: self.apply(variables, *a, **k), tokens, mask, 2 * (S - 1), self.min_prefix)
        lp = sequence_logprob(logits, tokens, mask).view(-1, 2)
        return lp[:, 0], lp[:, 1]

    def loss(self, variables, batch, step: Step):
        ref = step.ema if step.ema is not None else variables
        if self.share_prefix:
            pc, pr = self._pair_lp(variables, batch)
            with torch.no_grad():
                rc, rr = self._pair_lp(ref, batch)
        else:
            pc, pr = self._lp(variables, batch["chosen"], batch["chosen_mask"]), self._lp(variables, batch["rejected"], batch["rejected_mask"])
            with torch.no_grad():
                rc, rr = self._lp(ref, batch["chosen"], batch["chosen_mask"]), self._lp(ref, batch["rejected"], batch["rejected_mask"])
        margin = self.beta * ((pc - rc) - (pr - rr))
        per = -(1 - self.label_smoothing) * F.logsigmoid(margin) - self.label_smoothing * F.logsigmoid(-margin)
        n = torch.tensor(float(per.shape[0]), device=per.device)
        aux = Aux(metrics={"reward_accuracy": Ratio((margin > 0).float().sum(), n), "reward_margin": Ratio(margin.detach().sum(), n)})
        return Ratio(per.sum(), n), aux
