"""Consistency training and a latent world-model objective.

``ConsistencyObjective`` (consistency training, no teacher): the denoiser at a noisier point must agree with an EMA copy
of itself at the adjacent less noisy point on the same trajectory; the boundary transform ``c_skip / c_out`` pins
``f(x, sigma_min) = x``.  ``WorldModelObjective``: encode observations, roll a latent dynamics model under the actions,
and predict next latents (stop-gradient targets), rewards and episode ends.

Reference: src/dew/objectives/diffusion/consistency.py, src/dew/diffusion/transforms.py (``ConsistencyBoundary``),
src/dew/objectives/world_model.py.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from .base import Aux, Objective, Ratio, Step


class ConsistencyObjective(Objective):
    def __init__(self, model, sigma_min: float = 0.002, sigma_max: float = 80.0, sigma_data: float = 0.5, rho: float = 7.0,
                 levels: int = 18, ema_decay: float = 0.999, sample_key: str = "sample"):
        self.model, self.smin, self.smax, self.sd, self.rho, self.levels = model, sigma_min, sigma_max, sigma_data, rho, levels
        self.ema_decay, self.sample_key = ema_decay, sample_key

    def sigmas(self, device) -> torch.Tensor:
        i = torch.arange(self.levels, device=device, dtype=torch.float32)
        a, b = self.smin ** (1 / self.rho), self.smax ** (1 / self.rho)
        return (a + i / (self.levels - 1) * (b - a)) ** self.rho

    def denoise(self, variables, x, sigma):
        """``f(x, sigma) = c_skip x + c_out F(c_in x, log sigma / 4)`` with the consistency boundary at ``sigma_min``."""
        s = sigma.view(-1, *([1] * (x.dim() - 1)))
        c_skip = self.sd ** 2 / ((s - self.smin) ** 2 + self.sd ** 2)
        c_out = self.sd * (s - self.smin) / torch.sqrt(s ** 2 + self.sd ** 2)
        c_in = 1 / torch.sqrt(s ** 2 + self.sd ** 2)
        return c_skip * x + c_out * self.apply(variables, c_in * x, torch.log(sigma) / 4).float()

    def loss(self, variables, batch, step: Step):
        x0 = batch[self.sample_key].float()
        rows = x0.shape[0]
        sig = self.sigmas(x0.device)
        idx = (step.sample("level", (1,), rows, kind="uniform").to(x0.device).view(-1) * (self.levels - 1)).long().clamp(0, self.levels - 2)
        noise = step.sample("noise", tuple(x0.shape[1:]), rows).to(x0.device)
        hi, lo = sig[idx + 1], sig[idx]
        e = lambda s: s.view(-1, *([1] * (x0.dim() - 1)))
        student = self.denoise(variables, x0 + e(hi) * noise, hi)
        with torch.no_grad():
            teacher_vars = step.ema if step.ema is not None else variables
            target = self.denoise(teacher_vars, x0 + e(lo) * noise, lo)
        per = ((student - target) ** 2).reshape(rows, -1).mean(1)
        return Ratio(per.sum(), torch.tensor(float(rows), device=per.device)), Aux()

    @torch.no_grad()
    def generate(self, variables, shape, generator=None, device="cpu", steps: int = 1):
        """One-step (or multistep: re-noise to a lower level and denoise again) generation."""
        x = torch.randn(shape, generator=generator).to(device) * self.smax
        sig = self.sigmas(device)
        order = torch.linspace(self.levels - 1, 0, steps + 1).long()[:-1]
        out = None
        for n, i in enumerate(order):
            s = sig[i].expand(shape[0])
            if n > 0:
                x = out + math.sqrt(max(float(sig[i]) ** 2 - self.smin ** 2, 0.0)) * torch.randn(shape, generator=generator).to(device)
            out = self.denoise(variables, x, s)
        return out


class WorldModelObjective(Objective):
    """``model`` exposes ``encode(obs) -> z``, ``dynamics(z, action) -> z_next``, ``reward(z, action) -> r`` and
    ``done(z) -> logit``; the batch holds ``obs [B, T+1, ...]``, ``action [B, T, A]``, ``reward [B, T]``, ``done [B, T]``."""

    def __init__(self, model, horizon: Optional[int] = None, reward_weight: float = 1.0, done_weight: float = 1.0, ema_decay: Optional[float] = None):
        self.model, self.horizon, self.rw, self.dw, self.ema_decay = model, horizon, reward_weight, done_weight, ema_decay

    def loss(self, variables, batch, step: Step):
        obs, act = batch["observation"], batch["action"]
        B, T = act.shape[:2]
        H = min(self.horizon or T, T)
        m = self.model
        z_all = m.encode(obs.reshape(B * (T + 1), *obs.shape[2:])).reshape(B, T + 1, -1)
        z = z_all[:, 0]
        lat = rew = don = 0.0
        for t in range(H):
            r_hat = m.reward(z, act[:, t]).reshape(B)
            z = m.dynamics(z, act[:, t])
            lat = lat + F.mse_loss(z, z_all[:, t + 1].detach(), reduction="none").mean(1)
            rew = rew + (r_hat - batch["reward"][:, t].float()) ** 2
            don = don + F.binary_cross_entropy_with_logits(m.done(z).reshape(B), batch["done"][:, t].float(), reduction="none")
        per = (lat + self.rw * rew + self.dw * don) / H
        mass = torch.tensor(float(B), device=per.device)
        return Ratio(per.sum(), mass), Aux(metrics={"latent_mse": Ratio((lat / H).sum(), mass), "reward_mse": Ratio((rew / H).sum(), mass)})


def lambda_returns(rewards: torch.Tensor, values: torch.Tensor, continues: torch.Tensor, lam: float = 0.95) -> torch.Tensor:
    """TD(lambda) targets along an imagined trajectory.  rewards, continues ``[H, B]`` (continues = gamma * (1 - done)),
    values ``[H + 1, B]`` (the last row bootstraps): ``G_t = r_t + c_t ((1 - lam) V_{t+1} + lam G_{t+1})``."""
    H = rewards.shape[0]
    out = [None] * H
    nxt = values[-1]
    for t in range(H - 1, -1, -1):
        nxt = rewards[t] + continues[t] * ((1 - lam) * values[t + 1] + lam * nxt)
        out[t] = nxt
    return torch.stack(out, 0)


class DreamerObjective(Objective):
    """Actor-critic learning in imagination (Dreamer): from encoded start states the actor's actions are rolled through the
    learned dynamics for ``horizon`` steps; the critic regresses the lambda-returns of predicted rewards (targets without
    gradient), and the actor ascends the same returns by backpropagating through the dynamics and reward models, with an
    entropy bonus.  ``model`` is a world model as in ``WorldModelObjective`` plus ``actor(z) -> (mean, log_std)`` and
    ``critic(z) -> value``; only actor and critic receive gradients here (the world model's outputs are used as fixed
    functions: its parameters are excluded by the caller's parameter groups or frozen).
    Reference: src/dew/objectives/rl/ (dreamer), src/dew/rl/skydreamer.py."""

    def __init__(self, model, horizon: int = 15, gamma: float = 0.99, lam: float = 0.95, entropy: float = 1e-3,
                 ema_decay: Optional[float] = None):
        self.model, self.horizon, self.gamma, self.lam, self.entropy, self.ema_decay = model, horizon, gamma, lam, entropy, ema_decay

    def imagine(self, z0: torch.Tensor, step: Step):
        m = self.model
        zs, rewards, conts, ents = [z0], [], [], []
        z = z0
        for t in range(self.horizon):
            mean, log_std = m.actor(z.detach() if t == 0 else z)
            std = log_std.clamp(-5, 2).exp()
            eps = step.sample(f"action_{t}", tuple(mean.shape[1:]), mean.shape[0]).to(mean.device)
            action = torch.tanh(mean + std * eps)                          # reparameterised draw
            rewards.append(m.reward(z, action).reshape(-1))
            z = m.dynamics(z, action)
            conts.append(self.gamma * (1 - torch.sigmoid(m.done(z).reshape(-1))))
            ents.append((log_std + 0.5 * math.log(2 * math.pi * math.e)).sum(-1))
            zs.append(z)
        return torch.stack(zs, 0), torch.stack(rewards, 0), torch.stack(conts, 0), torch.stack(ents, 0)

    def loss(self, variables, batch, step: Step):
        m = self.model
        obs = batch["observation"]
        with torch.no_grad():
            z0 = m.encode(obs.reshape(-1, *obs.shape[2:]) if obs.dim() > 2 and "action" in batch else obs)
        zs, rewards, conts, ents = self.imagine(z0, step)
        values = m.critic(zs.reshape(-1, zs.shape[-1])).reshape(zs.shape[0], -1)
        targets = lambda_returns(rewards, values.detach(), conts.detach(), self.lam)
        # discount weights: later imagined steps count less once an episode is likely over
        weights = torch.cumprod(torch.cat([torch.ones_like(conts[:1]), conts[:-1]], 0), 0).detach()
        actor_loss = -(weights * (lambda_returns(rewards, values.detach(), conts, self.lam) + self.entropy * ents)).mean(0)
        critic_loss = (weights * (values[:-1] - targets.detach()) ** 2).mean(0)
        per = actor_loss + critic_loss
        mass = torch.tensor(float(per.shape[0]), device=per.device)
        return Ratio(per.sum(), mass), Aux(metrics={"imagined_return": Ratio(targets[0].detach().sum(), mass),
                                                    "critic_loss": Ratio(critic_loss.detach().sum(), mass)})
