"""Advantage estimators: plain functions from a batch's rewards (and values) to its advantages.  They know nothing of a model,
an objective or a batch dict, so an objective combines them and a test checks them on fixed tensors.

``masked_mean / masked_var / masked_whiten``  reductions over the positions a mask keeps (1e-8 in every mean; unbiased variance)
``group_advantage``      GRPO: each reward less its group's mean, over the group's deviation (ddof 1) plus eps
``dr_grpo_advantage``    the same without the deviation (Dr. GRPO)
``rloo_advantage``       each reward less the mean of the rest of its group, ``g / (g - 1)`` times the centred reward
``gae_advantages``       generalized advantage estimates of ``[B, T]`` rewards and values under a response mask
``gae``                  those, whitened over the mask, with the unwhitened returns
``discounted_returns`` / ``generalized_advantages``  time-major ``[T, B]`` forms with episode ends, for environment rollouts

Reference: src/dew/rl/advantage.py (``masked_mean``, ``masked_whiten``, ``group_advantage``, ``group_normalised``,
``rloo_advantage``, ``gae_advantages``, ``gae``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

MEAN_EPS = 1e-8
GROUP_EPS = 1e-6


def masked_mean(x: torch.Tensor, mask: torch.Tensor, dim=None) -> torch.Tensor:
    """Mean over the kept positions.  Values outside the mask are replaced by zero before the sum, so a NaN there is ignored."""
    m = mask.to(x.dtype)
    kept = torch.where(mask.bool(), x, torch.zeros_like(x))
    if dim is None:
        return kept.sum() / (m.sum() + MEAN_EPS)
    return kept.sum(dim) / (m.sum(dim) + MEAN_EPS)


def masked_var(x: torch.Tensor, mask: torch.Tensor, unbiased: bool = True) -> torch.Tensor:
    mean = masked_mean(x, mask)
    var = masked_mean((x - mean) ** 2, mask)
    if unbiased:
        n = mask.sum()
        if int(n) < 2:
            raise ValueError("an unbiased variance needs at least two kept positions")
        var = var * (n / (n - 1))
    return var


def masked_whiten(x: torch.Tensor, mask: torch.Tensor, shift_mean: bool = True) -> torch.Tensor:
    """``x`` centred on its masked mean and scaled by its unbiased masked deviation (positions outside the mask are transformed
    too and left for the caller to drop)."""
    mean, var = masked_mean(x, mask), masked_var(x, mask)
    out = (x - mean) * torch.rsqrt(var + MEAN_EPS)
    return out if shift_mean else out + mean


def group_normalised(grouped: torch.Tensor, eps: float = GROUP_EPS, ddof: int = 1, scale: bool = True) -> torch.Tensor:
    """Each row of ``[groups, members]`` less its mean, over its deviation plus ``eps``."""
    centred = grouped - grouped.mean(1, keepdim=True)
    if not scale:
        return centred
    if grouped.shape[1] <= ddof:
        return centred                                                   # one member: no deviation to divide by
    return centred / (grouped.std(1, keepdim=True, correction=ddof) + eps)


def group_advantage(rewards: torch.Tensor, group: int, eps: float = GROUP_EPS) -> torch.Tensor:
    """``[B]`` rewards with ``group`` consecutive completions per prompt -> ``[B]`` group-relative advantages."""
    if rewards.shape[0] % group:
        raise ValueError(f"{rewards.shape[0]} rewards do not split into groups of {group}")
    return group_normalised(rewards.reshape(-1, group), eps).reshape(-1)


def dr_grpo_advantage(rewards: torch.Tensor, group: int) -> torch.Tensor:
    return group_normalised(rewards.reshape(-1, group), scale=False).reshape(-1)


def global_advantage(rewards: torch.Tensor, group: int, eps: float = GROUP_EPS) -> torch.Tensor:
    """REINFORCE++ with a group baseline: each reward less its group's mean, then divided by the standard deviation of those differences
    over the whole batch (one scale for every prompt, so an easy prompt's small spread is not blown up to unit variance)."""
    if rewards.shape[0] % group:
        raise ValueError(f"{rewards.shape[0]} rewards do not split into groups of {group}")
    centred = (rewards.reshape(-1, group) - rewards.reshape(-1, group).mean(1, keepdim=True)).reshape(-1)
    return centred / (centred.std(unbiased=False) + eps)


def rloo_advantage(rewards: torch.Tensor, group: int) -> torch.Tensor:
    if group < 2:
        raise ValueError("leave-one-out needs at least two completions per prompt")
    g = rewards.reshape(-1, group)
    rest = (g.sum(1, keepdim=True) - g) / (group - 1)
    return (g - rest).reshape(-1)


def gae_advantages(rewards: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, gamma: float = 1.0, lam: float = 1.0
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Unwhitened estimates for ``[B, T]`` token rewards and values under a response mask: the recursion runs backwards from
    the last step with ``delta_t = r_t + gamma V_{t+1} - V_t`` and ``A_t = delta_t + gamma lam A_{t+1}``; a masked position
    passes its successor's value and advantage through unchanged.  Returns (advantages, returns = advantages + values)."""
    B, T = rewards.shape
    m = mask.to(rewards.dtype)
    adv = torch.zeros_like(rewards)
    next_value = torch.zeros_like(rewards[:, 0])
    run = torch.zeros_like(rewards[:, 0])
    for t in range(T - 1, -1, -1):
        delta = rewards[:, t] + gamma * next_value - values[:, t]
        step = delta + gamma * lam * run
        next_value = values[:, t] * m[:, t] + (1 - m[:, t]) * next_value
        run = step * m[:, t] + (1 - m[:, t]) * run
        adv[:, t] = run
    return adv, adv + values


def gae(rewards, values, mask, gamma: float = 1.0, lam: float = 1.0):
    adv, returns = gae_advantages(rewards, values, mask, gamma, lam)
    return masked_whiten(adv, mask) * mask.to(adv.dtype), returns


# ------------------------------------------------------------------------------------------------ time-major, with episode ends
def discounted_returns(rewards: torch.Tensor, dones: torch.Tensor, gamma: float, bootstrap: Optional[torch.Tensor] = None) -> torch.Tensor:
    T = rewards.shape[0]
    out = torch.zeros_like(rewards)
    run = torch.zeros_like(rewards[0]) if bootstrap is None else bootstrap.clone()
    for t in range(T - 1, -1, -1):
        run = rewards[t] + gamma * run * (1 - dones[t].float())
        out[t] = run
    return out


def generalized_advantages(rewards, values, dones, gamma: float = 0.99, lam: float = 0.95, bootstrap=None):
    """GAE(lambda) over ``[T, B]``: ``bootstrap [B]`` is the value after the last step; returns (advantages, returns)."""
    T = rewards.shape[0]
    nxt = torch.zeros_like(values[0]) if bootstrap is None else bootstrap
    adv = torch.zeros_like(rewards)
    run = torch.zeros_like(rewards[0])
    for t in range(T - 1, -1, -1):
        live = 1 - dones[t].float()
        delta = rewards[t] + gamma * nxt * live - values[t]
        run = delta + gamma * lam * live * run
        adv[t] = run
        nxt = values[t]
    return adv, adv + values


def lambda_returns(rewards: torch.Tensor, values: torch.Tensor, continues: torch.Tensor, lam: float = 0.95) -> torch.Tensor:
    """DreamerV3's bootstrapped lambda-returns over imagined ``[T, B]`` steps: ``R_t = r_t + c_t ((1 - lam) V_{t+1} + lam R_{t+1})``
    with ``R_T = V_T``; ``continues`` already holds the discount.  Returns ``[T - 1, B]``."""
    T = rewards.shape[0]
    out = []
    run = values[-1]
    for t in range(T - 2, -1, -1):
        run = rewards[t + 1] + continues[t + 1] * ((1 - lam) * values[t + 1] + lam * run)
        out.append(run)
    return torch.stack(out[::-1])
