"""PPO for continuous control in a batched functional ``Env``: a Gaussian actor (state-independent log-std, optionally squashed by
tanh with the Jacobian in its log-density) and a critic, rollouts of ``steps`` steps over ``envs`` environments with in-place restarts,
GAE that tells a terminal state (value zero) from a time limit (the cut state's value stands, read from the step's own final
observation), and the clipped surrogate with a clipped value loss over shuffled minibatches for a few epochs.  Observations are
normalised by running moments gathered from the rollouts.

Reference: src/dew/objectives/rl/control.py, src/dew/rl/env.py (``env_rollout``), src/dew/objectives/rl/ppo.py (clipped value loss, episode GAE).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ...rl.distributions import normal_entropy, normal_log_density, tanh_log_jacobian
from ...rl.env import Carry, Env, env_rollout, start, views


def flat_observation(observation) -> torch.Tensor:
    """An observation's views side by side (in the order of their names), one vector per environment; leading axes are kept."""
    parts = views(observation)
    names = sorted(parts)
    if len(names) == 1:
        return parts[names[0]].float()
    batch = min(v.dim() for v in parts.values()) - 1
    return torch.cat([parts[n].float().reshape(*parts[n].shape[:batch], -1) for n in names], -1)


def episode_gae(rewards, values, next_values, terminated, done, gamma: float = 0.99, lam: float = 0.95) -> Tuple[torch.Tensor, torch.Tensor]:
    """``[T, N]`` inputs; ``next_values[t]`` is the critic on the observation step ``t`` ended in (before any restart).  A terminal step
    bootstraps nothing; a truncated step bootstraps its own final state and stops the accumulation.  Returns (advantages, returns)."""
    T = rewards.shape[0]
    adv = torch.zeros_like(rewards)
    run = torch.zeros_like(rewards[0])
    for t in range(T - 1, -1, -1):
        delta = rewards[t] + gamma * next_values[t] * (~terminated[t]).float() - values[t]
        run = delta + gamma * lam * (~done[t]).float() * run
        adv[t] = run
    return adv, adv + values


class RunningMoments(nn.Module):
    def __init__(self, size: int, eps: float = 1e-4):
        super().__init__()
        self.register_buffer("mean", torch.zeros(size))
        self.register_buffer("var", torch.ones(size))
        self.register_buffer("count", torch.tensor(eps))

    @torch.no_grad()
    def update(self, x: torch.Tensor) -> None:
        x = x.reshape(-1, x.shape[-1]).float()
        n = x.shape[0]
        mean, var = x.mean(0), x.var(0, unbiased=False)
        delta, total = mean - self.mean, self.count + n
        self.var.copy_((self.var * self.count + var * n + delta ** 2 * self.count * n / total) / total)
        self.mean.add_(delta * n / total)
        self.count.copy_(total)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ((x - self.mean) / torch.sqrt(self.var + 1e-8)).clamp(-10, 10)


def _mlp(sizes: Sequence[int], out_gain: float) -> nn.Sequential:
    layers: List[nn.Module] = []
    for i, (a, b) in enumerate(zip(sizes[:-1], sizes[1:])):
        lin = nn.Linear(a, b)
        nn.init.orthogonal_(lin.weight, gain=out_gain if i == len(sizes) - 2 else math.sqrt(2))
        nn.init.zeros_(lin.bias)
        layers += [lin] + ([nn.Tanh()] if i < len(sizes) - 2 else [])
    return nn.Sequential(*layers)


class ActorCritic(nn.Module):
    def __init__(self, observation_size: int, action_size: int, hidden: Sequence[int] = (64, 64), squash: bool = True, initial_std: float = 0.6):
        super().__init__()
        self.squash = squash
        self.moments = RunningMoments(observation_size)
        self.actor = _mlp([observation_size, *hidden, action_size], 0.01)
        self.critic = _mlp([observation_size, *hidden, 1], 1.0)
        self.log_std = nn.Parameter(torch.full((action_size,), math.log(initial_std)))

    def distribution(self, obs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        x = self.moments(obs.float())
        return self.actor(x), self.log_std.exp().expand(obs.shape[0], -1), self.critic(x).squeeze(-1)

    def log_prob(self, raw: torch.Tensor, mean: torch.Tensor, std: torch.Tensor) -> torch.Tensor:
        lp = normal_log_density(raw, mean, std).sum(-1)
        return lp - tanh_log_jacobian(raw).sum(-1) if self.squash else lp

    def act(self, obs: torch.Tensor, key: Optional[int] = None, greedy: bool = False):
        mean, std, value = self.distribution(obs)
        if greedy:
            raw = mean
        else:
            g = torch.Generator(device="cpu").manual_seed(int(key))
            raw = mean + std * torch.randn(mean.shape, generator=g).to(mean.device)
        action = torch.tanh(raw) if self.squash else raw
        return action, {"raw": raw, "log_prob": self.log_prob(raw, mean, std), "value": value}

    def policy(self, params, observation, memory, key):
        """The ``dew_b200.rl.env.Policy`` signature (``params`` unused: the module holds its own)."""
        with torch.no_grad():
            action, extras = self.act(flat_observation(observation), key)
        return action, extras, memory


class ControlPPO:
    def __init__(self, env: Env, model: ActorCritic, envs: int = 64, steps: int = 64, epochs: int = 4, minibatches: int = 4, clip: float = 0.2,
                 gamma: float = 0.99, lam: float = 0.95, value_coef: float = 0.5, entropy_coef: float = 0.0, value_clip: Optional[float] = 0.2,
                 learning_rate: float = 3e-4, max_grad_norm: float = 0.5, seed: int = 0, normalize_advantages: bool = True):
        self.env, self.model = env, model
        self.envs, self.steps, self.epochs, self.minibatches = envs, steps, epochs, minibatches
        self.clip, self.gamma, self.lam, self.value_coef, self.entropy_coef, self.value_clip = clip, gamma, lam, value_coef, entropy_coef, value_clip
        self.max_grad_norm, self.normalize_advantages = max_grad_norm, normalize_advantages
        self.optimizer = torch.optim.Adam(model.parameters(), lr=learning_rate, eps=1e-5)
        self.carry: Carry = start(env, seed, envs)
        self.generator = torch.Generator().manual_seed(seed)
        self._returns = torch.zeros(envs)
        self.finished: List[float] = []

    # ------------------------------------------------------------------ data
    def collect(self) -> Dict[str, torch.Tensor]:
        self.carry, tr = env_rollout(self.env, self.model.policy, None, self.carry, self.steps)
        obs, nxt = flat_observation(tr.observation), flat_observation(tr.step.observation)
        self.model.moments.update(obs)
        with torch.no_grad():
            T, N = obs.shape[:2]
            _, _, values = self.model.distribution(obs.reshape(T * N, -1))
            _, _, next_values = self.model.distribution(nxt.reshape(T * N, -1))
            values, next_values = values.view(T, N), next_values.view(T, N)
            # the log-probabilities the rollout recorded were taken under the moments before this update: take them again
            mean, std, _ = self.model.distribution(obs.reshape(T * N, -1))
            old_lp = self.model.log_prob(tr.extras["raw"].reshape(T * N, -1), mean, std).view(T, N)
            adv, ret = episode_gae(tr.step.reward.float(), values, next_values, tr.step.terminated, tr.step.done, self.gamma, self.lam)
        for t in range(T):                                        # episodic returns, for the learning curve
            self._returns += tr.step.reward[t].float().cpu()
            ended = tr.step.done[t].cpu()
            self.finished += self._returns[ended].tolist()
            self._returns[ended] = 0.0
        flat = lambda x: x.reshape(T * N, *x.shape[2:])
        return {"observation": flat(obs), "raw": flat(tr.extras["raw"]), "old_log_prob": flat(old_lp), "old_value": flat(values), "advantage": flat(adv),
                "return": flat(ret)}

    # ------------------------------------------------------------------ update
    def loss(self, batch: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, Dict[str, float]]:
        mean, std, value = self.model.distribution(batch["observation"])
        lp = self.model.log_prob(batch["raw"], mean, std)
        adv = batch["advantage"]
        if self.normalize_advantages:
            adv = (adv - adv.mean()) / (adv.std(unbiased=False) + 1e-8)
        ratio = (lp - batch["old_log_prob"]).exp()
        policy = -torch.minimum(ratio * adv, ratio.clamp(1 - self.clip, 1 + self.clip) * adv).mean()
        err = (value - batch["return"]) ** 2
        if self.value_clip is not None:
            clipped = batch["old_value"] + (value - batch["old_value"]).clamp(-self.value_clip, self.value_clip)
            err = torch.maximum(err, (clipped - batch["return"]) ** 2)
        value_loss = 0.5 * err.mean()
        entropy = normal_entropy(std).sum(-1).mean()
        total = policy + self.value_coef * value_loss - self.entropy_coef * entropy
        return total, {"policy_loss": float(policy.detach()), "value_loss": float(value_loss.detach()), "entropy": float(entropy.detach()),
                       "clip_fraction": float(((ratio.detach() - 1).abs() > self.clip).float().mean()), "approx_kl": float((batch["old_log_prob"] - lp).mean().detach())}

    def update(self, batch: Dict[str, torch.Tensor]) -> Dict[str, float]:
        n = batch["observation"].shape[0]
        size = n // self.minibatches
        metrics: Dict[str, float] = {}
        for _ in range(self.epochs):
            order = torch.randperm(n, generator=self.generator)
            for j in range(self.minibatches):
                idx = order[j * size:(j + 1) * size].to(batch["observation"].device)
                loss, metrics = self.loss({k: v[idx] for k, v in batch.items()})
                self.optimizer.zero_grad(set_to_none=True)
                loss.backward()
                nn.utils.clip_grad_norm_(self.model.parameters(), self.max_grad_norm)
                self.optimizer.step()
        return metrics

    def train(self, iterations: int) -> List[Dict[str, float]]:
        history = []
        for _ in range(iterations):
            seen = len(self.finished)
            metrics = self.update(self.collect())
            recent = self.finished[seen:]
            metrics["episodes"] = float(len(recent))
            metrics["episode_return"] = float(sum(recent) / len(recent)) if recent else float("nan")
            history.append(metrics)
        return history
