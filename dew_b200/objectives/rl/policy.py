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
    starts_from_model = True
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
    starts_from_model = True
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


class FlowGRPO(Objective):
    starts_from_model = True
    """GRPO for flow-matching samplers (Flow-GRPO): the ODE sampler is turned into an SDE with the same marginals so that
    every denoising step is a Gaussian policy, ``x_{t-dt} ~ N(mean_theta(x_t, t), sigma_t^2 dt)``; images sampled in groups from
    one prompt are rewarded, rewards are whitened inside the group, and the clipped policy-gradient ratio is taken per
    step from the Gaussian log-densities (old policy = the sampler that produced the trajectory), with an optional KL
    pull towards a frozen reference velocity.  ``batch``: ``x [rows, steps + 1, ...]`` the stored trajectory, ``t [steps + 1]`` its
    time grid (1 -> 0), ``old_logp [rows, steps]``, ``rewards [rows]``.  The model is called as ``model(x, t)`` -> velocity.
    Reference: src/dew/objectives/rl/ (FlowGRPO)."""

    def __init__(self, model, group: int = 4, clip: float = 0.2, noise_level: float = 0.7, kl_weight: float = 0.0, reference=None):
        self.model, self.group, self.clip, self.a, self.kl_weight, self.reference = model, group, clip, noise_level, kl_weight, reference
        self.ema_decay = None

    def step_distribution(self, variables, x, t, dt):
        """Mean and standard deviation of the SDE step from ``t`` to ``t - dt`` on the path ``x_t = (1 - t) x_0 + t eps``."""
        tt = t.clamp(1e-3, 1 - 1e-3)
        v = self.apply(variables, x, t.expand(x.shape[0])).float()
        sigma = self.a * torch.sqrt(tt / (1 - tt))
        # score of the marginal expressed through the velocity: x_0 = x - t v, eps = x + (1 - t) v
        drift = v + (sigma ** 2 / (2 * tt)) * (x + (1 - tt) * v)
        mean = x - drift * dt
        return mean, sigma * torch.sqrt(dt), v

    def logp(self, variables, x_t, x_next, t, dt):
        mean, std, v = self.step_distribution(variables, x_t, t, dt)
        lp = -0.5 * (((x_next - mean) / std) ** 2).reshape(x_t.shape[0], -1).sum(1) - x_t[0].numel() * torch.log(std)
        return lp, v

    @torch.no_grad()
    def rollout(self, variables, shape, steps: int, generator=None, device="cpu"):
        """Sample trajectories with the SDE sampler: returns ``x [rows, steps + 1, ...]``, the time grid and ``old_logp``."""
        x = torch.randn(shape, generator=generator).to(device)
        grid = torch.linspace(1.0, 0.0, steps + 1, device=device)
        xs, lps = [x], []
        for i in range(steps):
            t, dt = grid[i], grid[i] - grid[i + 1]
            mean, std, _ = self.step_distribution(variables, x, t, dt)
            x = mean + std * torch.randn(shape, generator=generator).to(device)
            lp, _ = self.logp(variables, xs[-1], x, t, dt)
            xs.append(x)
            lps.append(lp)
        return torch.stack(xs, 1), grid, torch.stack(lps, 1)

    def loss(self, variables, batch, step: Step):
        x, grid, old, rewards = batch["x"].float(), batch["t"].float(), batch["old_logp"].float(), batch["rewards"].float()
        rows, steps = old.shape
        adv = group_advantages(rewards, self.group)
        total = x.new_zeros(())
        kl = x.new_zeros(())
        for i in range(steps):
            t, dt = grid[i], grid[i] - grid[i + 1]
            lp, v = self.logp(variables, x[:, i], x[:, i + 1], t, dt)
            ratio = torch.exp(lp - old[:, i])
            surr = torch.minimum(ratio * adv, ratio.clamp(1 - self.clip, 1 + self.clip) * adv)
            total = total - surr.sum()
            if self.kl_weight and self.reference is not None:
                with torch.no_grad():
                    v_ref = self.reference(x[:, i], t.expand(rows)).float()
                kl = kl + ((v - v_ref) ** 2).reshape(rows, -1).mean(1).sum()
        total = total + self.kl_weight * kl
        mass = torch.tensor(float(rows * steps), device=x.device)
        return Ratio(total, mass), Aux(metrics={"reward": Ratio(rewards.sum(), torch.tensor(float(rows), device=x.device))})
