"""DiffusionNFT (arXiv 2509.16117): online reinforcement of a flow model on the *forward* process.  Images are sampled from the old
policy with any solver (no stochastic sampler, no stored trajectories, no likelihoods), rewarded, and each reward is turned into an
optimality probability ``r`` in [0, 1] by normalising inside its prompt's group.  Training then draws a time and a noise for every image,
``x_t = (1 - t) x_0 + t eps`` with the flow-matching target ``v = eps - x_0``, and fits two implicit policies around the old one,

    v+ = (1 - beta) v_old + beta v_theta          the positive policy, trained on the image with weight r
    v- = (1 + beta) v_old - beta v_theta          the negative policy, trained on it with weight 1 - r

    loss = r |v+ - v|^2 + (1 - r) |v- - v|^2

so a well-rewarded image pulls ``v_theta`` towards reproducing it and a badly rewarded one pushes it away, by the same supervised
regression a flow model is pre-trained with.  The old policy is the trainer's weight average (``step.ema``), which follows the trained
weights by a soft update; before any average exists the trained weights stand in (the first step then has zero gradient difference
between the two policies and is plain reward-weighted regression).

``batch``: ``x0 [B, ...]`` sampled images (or latents), ``rewards [B]`` with ``group`` consecutive images per prompt, optional ``cond``
passed to the model as ``model(x, t, cond)``.

Reference: src/dew/objectives/rl/nft.py.
"""
from __future__ import annotations

from typing import Optional

import torch

from ...rl import advantage as A
from ..base import Aux, EMASpec, Objective, Ratio, Step


def optimality(rewards: torch.Tensor, group: int, spread: float = 1.0) -> torch.Tensor:
    """Rewards -> ``r`` in [0, 1]: half plus half the group-normalised reward over ``spread``, clipped."""
    return (0.5 + 0.5 * (A.group_advantage(rewards.float(), group) / spread).clamp(-1, 1))


class DiffusionNFT(Objective):
    starts_from_model = True

    def __init__(self, model, group: int = 4, beta: float = 1.0, spread: float = 1.0, old_decay: float = 0.9, t_min: float = 0.0, t_max: float = 1.0):
        if not 0 < beta:
            raise ValueError("beta is positive: it sets how far the implicit policies stand from the old one")
        self.model, self.group, self.beta, self.spread, self.t_min, self.t_max = model, group, beta, spread, t_min, t_max
        self.ema_decay = EMASpec.constant(old_decay)

    def velocity(self, variables, x, t, cond):
        out = self.apply(variables, x, t) if cond is None else self.apply(variables, x, t, cond)
        return (out[0] if isinstance(out, tuple) else out).float()

    def loss(self, variables, batch, step: Step):
        x0 = batch["x0"].float()
        B = x0.shape[0]
        r = optimality(batch["rewards"], self.group, self.spread).to(x0.device)
        t = self.t_min + (self.t_max - self.t_min) * step.sample("nft_t", (), B, kind="uniform").to(x0.device).float()
        eps = step.sample("nft_eps", tuple(x0.shape[1:]), B).to(x0.device).float()
        tb = t.view(B, *([1] * (x0.dim() - 1)))
        x_t, target = (1 - tb) * x0 + tb * eps, eps - x0
        cond = batch.get("cond")
        v = self.velocity(variables, x_t, t, cond)
        with torch.no_grad():
            v_old = self.velocity(step.ema, x_t, t, cond) if step.ema is not None else v.detach()
        pos = ((1 - self.beta) * v_old + self.beta * v - target).pow(2).reshape(B, -1).mean(1)
        neg = ((1 + self.beta) * v_old - self.beta * v - target).pow(2).reshape(B, -1).mean(1)
        total = (r * pos + (1 - r) * neg).sum()
        mass = torch.tensor(float(B), device=x0.device)
        metrics = {"reward": Ratio(batch["rewards"].float().sum().to(x0.device), mass), "optimality": Ratio(r.sum(), mass),
                   "policy_gap": Ratio((v.detach() - v_old).pow(2).reshape(B, -1).mean(1).sum(), mass)}
        return Ratio(total, mass), Aux(metrics=metrics)
