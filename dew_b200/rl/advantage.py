"""Returns and generalized advantage estimates over ``[T, B]`` rollouts.  Reference: src/dew/rl/advantage.py."""
from __future__ import annotations

import torch


def discounted_returns(rewards: torch.Tensor, dones: torch.Tensor, gamma: float, bootstrap: torch.Tensor | None = None) -> torch.Tensor:
    T = rewards.shape[0]
    out = torch.zeros_like(rewards)
    run = torch.zeros_like(rewards[0]) if bootstrap is None else bootstrap.clone()
    for t in range(T - 1, -1, -1):
        run = rewards[t] + gamma * run * (1 - dones[t].float())
        out[t] = run
    return out


def generalized_advantages(rewards, values, dones, gamma: float = 0.99, lam: float = 0.95, bootstrap=None):
    """GAE(lambda): ``values [T, B]``, ``bootstrap [B]`` the value after the last step; returns (advantages, returns)."""
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
