"""Policy-gradient objectives over sampled completions: ``GRPO`` (group-relative advantages, clipped ratio, KL to the
reference in the EMA slot) and ``PPO`` (clipped surrogate + value loss + entropy bonus).
Reference: src/dew/objectives/rl (GRPO, PPO), src/dew/rl/advantage.py."""
from __future__ import annotations

import torch

from ..base import Aux, EMASpec, Objective, Ratio, Step


def group_advantages(rewards: torch.Tensor, group: int, eps: float = 1e-6) -> torch.Tensor:
    """Standardise rewards within each group of ``group`` completions of the same prompt."""
    r = rewards.float().reshape(-1, group)
    return ((r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True) + eps)).reshape(-1)


def gae(rewards, values, dones, gamma: float = 0.99, lam: float = 0.95):
    """Generalised advantage estimation over ``[T, B]`` trajectories; ``values`` has one extra bootstrap row."""
    T = rewards.shape[0]
    adv = torch.zeros_like(rewards)
    last = torch.zeros_like(rewards[0])
    for t in reversed(range(T)):
        nonterminal = 1.0 - dones[t].float()
        delta = rewards[t] + gamma * values[t + 1] * nonterminal - values[t]
        last = delta + gamma * lam * nonterminal * last
        adv[t] = last
    return adv, adv + values[:-1]


def _token_logprobs(logits, tokens):
    return torch.log_softmax(logits.float(), -1).gather(-1, tokens[:, 1:, None]).squeeze(-1)


class GRPO(Objective):
    """batch: ``tokens [B,S]``, ``mask [B,S]`` (1 on completion tokens), ``rewards [B]``, ``old_logprobs [B,S-1]``."""

    def __init__(self, model, group: int = 4, clip: float = 0.2, kl: float = 0.04):
        self.model, self.group, self.clip, self.kl = model, group, clip, kl
        self.ema_decay = EMASpec.constant(1.0)

    def loss(self, variables, batch, step: Step):
        tokens, mask = batch["tokens"], batch["mask"][:, 1:].float()
        lp = _token_logprobs(self.apply(variables, tokens[:, :-1]), tokens)
        adv = group_advantages(batch["rewards"], self.group).to(lp.device)[:, None]
        ratio = torch.exp(lp - batch["old_logprobs"].float())
        surr = torch.minimum(ratio * adv, ratio.clamp(1 - self.clip, 1 + self.clip) * adv)
        per = -surr
        aux_metrics = {}
        if self.kl and step.ema is not None:
            with torch.no_grad():
                ref = _token_logprobs(self.apply(step.ema, tokens[:, :-1]), tokens)
            d = ref - lp
            klv = torch.exp(d) - d - 1                                 # the k3 estimator
            per = per + self.kl * klv
            aux_metrics["kl"] = Ratio((klv.detach() * mask).sum(), mask.sum())
        aux_metrics["clip_fraction"] = Ratio((((ratio - 1).abs() > self.clip).float() * mask).sum(), mask.sum())
        return Ratio((per * mask).sum(), mask.sum()), Aux(metrics=aux_metrics)


class PPO(Objective):
    """The model returns ``(logits, values)``; batch: ``tokens, mask, advantages [B,S-1], returns [B,S-1], old_logprobs``."""

    def __init__(self, model, clip: float = 0.2, value_coef: float = 0.5, entropy_coef: float = 0.0):
        self.model, self.clip, self.value_coef, self.entropy_coef = model, clip, value_coef, entropy_coef

    def loss(self, variables, batch, step: Step):
        tokens, mask = batch["tokens"], batch["mask"][:, 1:].float()
        logits, values = self.apply(variables, tokens[:, :-1])
        lp = _token_logprobs(logits, tokens)
        ratio = torch.exp(lp - batch["old_logprobs"].float())
        adv = batch["advantages"].float()
        policy = -torch.minimum(ratio * adv, ratio.clamp(1 - self.clip, 1 + self.clip) * adv)
        value = 0.5 * (values.float().squeeze(-1) - batch["returns"].float()) ** 2
        p = torch.softmax(logits.float(), -1)
        ent = -(p * torch.log(p.clamp_min(1e-12))).sum(-1)
        per = policy + self.value_coef * value - self.entropy_coef * ent
        m = mask.sum()
        return Ratio((per * mask).sum(), m), Aux(metrics={"entropy": Ratio((ent.detach() * mask).sum(), m),
                                                           "value_loss": Ratio((value.detach() * mask).sum(), m)})
