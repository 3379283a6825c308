"""DreamerV3 (arXiv 2301.04104): a recurrent state-space world model learned from replayed experience, and an actor and a critic
learned inside its imagination.

World model: a GRU carries the deterministic state ``h``; the stochastic state ``z`` is ``stoch`` categoricals of ``classes`` classes
(1 % uniform mix, straight-through one-hot draws).  The prior reads ``h`` alone, the posterior ``h`` and the encoded observation.
Heads on ``(h, z)``: a decoder (symlog mean-squared error), a reward head and a critic (two-hot over bins evenly spaced in symlog space), a
continuation head (Bernoulli).  Loss: prediction + 0.5 x KL(sg(post) || prior) + 0.1 x KL(post || sg(prior)), both KLs clipped below
at one nat (free bits).  Behaviour: from every replayed posterior state the actor's actions are rolled ``horizon`` steps through
the prior; lambda-returns bootstrap from the critic; returns are scaled by an EMA of their 5th-95th percentile range (never below
1); the actor ascends ``sg(advantage / scale) log pi + eta entropy`` (REINFORCE), the critic regresses the lambda-returns and
stays near its own slow (EMA) copy.

A batch is a window of steps as ``rl.env.Driven`` / ``rl.simulator.DrivenSimulator`` record them: ``observation [B, T, ...]`` (or the
named views), ``action [B, T, A]`` (the action that led to the step), ``reward``, ``first``, ``last``, ``terminal``.  ``DreamerPolicy``
acts in an ``Env`` carrying ``(h, z, previous action)`` as its memory; ``DreamerRollout`` collects steps into a ``ReplayBuffer``
(with a teacher's labels when given: ``rl.aggregation``).

Reference: src/dew/objectives/rl/dreamer.py (world model, imagination, ``DreamerRollout``), src/dew/rl/distributions.py.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...rl import distributions as D
from ...rl.advantage import lambda_returns
from ...rl.env import Carry, Driven, Env, env_rollout, start, views
from ...rl.replay import ReplayBuffer
from ..base import Aux, Objective, Ratio, Step


def _mlp(inp: int, hidden: int, out: int, layers: int = 2) -> nn.Sequential:
    mods, d = [], inp
    for _ in range(layers):
        mods += [nn.Linear(d, hidden), nn.LayerNorm(hidden), nn.SiLU()]
        d = hidden
    mods.append(nn.Linear(d, out))
    return nn.Sequential(*mods)


class RSSM(nn.Module):
    def __init__(self, embed: int, action: int, deter: int = 128, stoch: int = 8, classes: int = 8, hidden: int = 128, unimix: float = 0.01):
        super().__init__()
        self.deter, self.stoch, self.classes, self.unimix = deter, stoch, classes, unimix
        self.inp = nn.Sequential(nn.Linear(stoch * classes + action, hidden), nn.LayerNorm(hidden), nn.SiLU())
        self.gru = nn.GRUCell(hidden, deter)
        self.prior = _mlp(deter, hidden, stoch * classes, 1)
        self.post = _mlp(deter + embed, hidden, stoch * classes, 1)

    @property
    def features(self) -> int:
        return self.deter + self.stoch * self.classes

    def initial(self, n: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        return torch.zeros(n, self.deter, device=device), torch.zeros(n, self.stoch * self.classes, device=device)

    def _logp(self, logits: torch.Tensor) -> torch.Tensor:
        return D.unimix_log_probs(logits.reshape(*logits.shape[:-1], self.stoch, self.classes), self.unimix)

    def _draw(self, logp: torch.Tensor, generator=None, mode: bool = False) -> torch.Tensor:
        if mode:                                                           # the most likely class of each categorical (deterministic acting)
            return F.one_hot(logp.argmax(-1), self.classes).to(logp.dtype).reshape(*logp.shape[:-2], self.stoch * self.classes)
        return D.onehot_sample(logp, generator).reshape(*logp.shape[:-2], self.stoch * self.classes)

    def img_step(self, h, z, action, generator=None):
        h = self.gru(self.inp(torch.cat([z, action], -1)), h)
        prior = self._logp(self.prior(h))
        return h, self._draw(prior, generator), prior

    def obs_step(self, h, z, action, embed, first, generator=None, mode: bool = False):
        keep = (~first).to(h.dtype)[:, None]                               # an episode's first step starts from the zero state
        h, z, action = h * keep, z * keep, action * keep
        h = self.gru(self.inp(torch.cat([z, action], -1)), h)
        prior = self._logp(self.prior(h))
        post = self._logp(self.post(torch.cat([h, embed], -1)))
        return h, self._draw(post, generator, mode), prior, post


class DreamerModel(nn.Module):
    """Vector observations (one view or several concatenated); continuous actions in [-1, 1] (a tanh-squashed normal) or a
    categorical over ``action`` choices when ``discrete``."""

    def __init__(self, observation: int, action: int, discrete: bool = False, deter: int = 128, stoch: int = 8, classes: int = 8, hidden: int = 128,
                 bins: int = 255):
        super().__init__()
        self.discrete, self.action_size = discrete, action
        self.encoder = _mlp(observation, hidden, hidden, 2)
        self.rssm = RSSM(hidden, action, deter, stoch, classes, hidden)
        f = self.rssm.features
        self.decoder = _mlp(f, hidden, observation, 2)
        self.reward = _mlp(f, hidden, bins, 2)
        self.cont = _mlp(f, hidden, 1, 2)
        self.actor = _mlp(f, hidden, action if discrete else 2 * action, 2)
        self.critic = _mlp(f, hidden, bins, 2)
        self.slow_critic = _mlp(f, hidden, bins, 2)
        self.slow_critic.load_state_dict(self.critic.state_dict())
        for p in self.slow_critic.parameters():
            p.requires_grad_(False)
        for head in (self.reward, self.critic):
            nn.init.zeros_(head[-1].weight)                                # zero-initialised output layers: predictions start at zero
            nn.init.zeros_(head[-1].bias)
        # evenly spaced bins in symlog space (the paper's symlog two-hot): a prediction is symexp of the bins' expectation, which a
        # little stray probability on the outermost bins moves by a little - with symexp-spaced bins it would move it by 1e8
        self.register_buffer("bins", torch.linspace(-20.0, 20.0, bins))
        self.register_buffer("return_range", torch.ones(()))

    def feat(self, h, z):
        return torch.cat([h, z], -1)

    def act(self, feat: torch.Tensor, generator=None, greedy: bool = False):
        """-> (action, log-probability, entropy)."""
        out = self.actor(feat)
        if self.discrete:
            logp = D.unimix_log_probs(out, 0.01)
            a = F.one_hot(logp.argmax(-1), self.action_size).to(feat.dtype) if greedy else D.onehot_sample(logp, generator).detach()
            return a, (logp * a).sum(-1), -(logp.exp() * logp).sum(-1)
        mean, raw_std = out.chunk(2, -1)
        std = 0.1 + 0.9 * torch.sigmoid(raw_std + 2.0)                      # bounded scale
        eps = torch.zeros_like(mean) if greedy else torch.randn(mean.shape, generator=generator).to(mean.device)
        raw = (mean + std * eps).detach()
        a = torch.tanh(raw)
        logp = (D.normal_log_density(raw, mean, std) - D.tanh_log_jacobian(raw)).sum(-1)
        return a, logp, D.normal_entropy(std).sum(-1)

    def value(self, feat, slow: bool = False) -> torch.Tensor:
        return D.symexp(D.twohot_mean((self.slow_critic if slow else self.critic)(feat), self.bins))


def flat_observation(batch: Mapping[str, torch.Tensor], names: Optional[Sequence[str]] = None) -> torch.Tensor:
    if names is None:
        return batch["observation"].float()
    return torch.cat([batch[n].float() for n in names], -1)


class DreamerV3(Objective):
    def __init__(self, model: DreamerModel, horizon: int = 15, gamma: float = 0.997, lam: float = 0.95, entropy: float = 3e-4, free_bits: float = 1.0,
                 dyn_scale: float = 0.5, rep_scale: float = 0.1, slow_decay: float = 0.98, slow_reg: float = 1.0, views: Optional[Sequence[str]] = None,
                 imitation: float = 0.0, ema_decay=None):
        self.model, self.horizon, self.gamma, self.lam, self.entropy = model, horizon, gamma, lam, entropy
        self.free_bits, self.dyn_scale, self.rep_scale = free_bits, dyn_scale, rep_scale
        self.slow_decay, self.slow_reg, self.views, self.imitation, self.ema_decay = slow_decay, slow_reg, views, imitation, ema_decay

    # ------------------------------------------------------------------ the world model over a replayed window
    def observe(self, batch, generator=None):
        m = self.model
        obs = D.symlog(flat_observation(batch, self.views))
        B, T = obs.shape[:2]
        embed = m.encoder(obs)
        action = batch["action"].float()
        first = batch["first"].bool()
        h, z = m.rssm.initial(B, obs.device)
        hs, zs, priors, posts = [], [], [], []
        for t in range(T):
            h, z, prior, post = m.rssm.obs_step(h, z, action[:, t], embed[:, t], first[:, t], generator)
            hs.append(h); zs.append(z); priors.append(prior); posts.append(post)
        return torch.stack(hs, 1), torch.stack(zs, 1), torch.stack(priors, 1), torch.stack(posts, 1), obs

    def world_model_loss(self, batch, generator=None):
        m = self.model
        hs, zs, priors, posts, obs = self.observe(batch, generator)
        feat = m.feat(hs, zs)
        recon = ((m.decoder(feat) - obs) ** 2).sum(-1)
        reward = D.twohot_loss(m.reward(feat), D.symlog(batch["reward"].float()), m.bins)
        cont_target = 1.0 - batch["terminal"].float()
        cont = F.binary_cross_entropy_with_logits(m.cont(feat).squeeze(-1), cont_target, reduction="none")
        dyn = D.categorical_kl(posts.detach(), priors).sum(-1).clamp_min(self.free_bits)
        rep = D.categorical_kl(posts, priors.detach()).sum(-1).clamp_min(self.free_bits)
        per = recon + reward + cont + self.dyn_scale * dyn + self.rep_scale * rep
        metrics = {"recon": recon.detach().mean(), "reward_loss": reward.detach().mean(), "cont_loss": cont.detach().mean(),
                   "kl": D.categorical_kl(posts, priors).sum(-1).detach().mean()}
        return per, feat, hs, zs, metrics

    # ------------------------------------------------------------------ behaviour in imagination
    def imagine(self, h, z, generator=None):
        m = self.model
        feats, logps, ents, actions = [m.feat(h, z)], [], [], []
        for _ in range(self.horizon):
            a, logp, ent = m.act(feats[-1].detach(), generator)
            with torch.no_grad():                                           # REINFORCE: nothing differentiates through the dynamics
                h, z, _ = m.rssm.img_step(h, z, a, generator)
            feats.append(m.feat(h, z)); logps.append(logp); ents.append(ent); actions.append(a)
        return torch.stack(feats), torch.stack(logps), torch.stack(ents)

    def behaviour_loss(self, hs, zs, generator=None):
        m = self.model
        h0, z0 = hs.detach().reshape(-1, hs.shape[-1]), zs.detach().reshape(-1, zs.shape[-1])
        feats, logps, ents = self.imagine(h0, z0, generator)
        feats = feats.detach()                                              # REINFORCE: no gradient through the dynamics
        with torch.no_grad():
            reward = D.symexp(D.twohot_mean(m.reward(feats), m.bins))      # [H + 1, N]
            cont = torch.sigmoid(m.cont(feats).squeeze(-1)) * self.gamma
            value = m.value(feats)                                           # raw units
            returns = lambda_returns(reward, value, cont, self.lam)         # [H, N]
            weights = torch.cumprod(torch.cat([torch.ones_like(cont[:1]), cont[:-1]]), 0)[:-1]
            lo, hi = torch.quantile(returns.flatten(), 0.05), torch.quantile(returns.flatten(), 0.95)
            m.return_range.mul_(0.99).add_(0.01 * (hi - lo))
            scale = m.return_range.clamp_min(1.0)
            advantage = (returns - value[:-1]) / scale
        actor = -(weights * (advantage * logps + self.entropy * ents)).mean()
        critic_logits = m.critic(feats[:-1])
        critic = D.twohot_loss(critic_logits, D.symlog(returns), m.bins)
        with torch.no_grad():
            slow = D.twohot(D.symlog(m.value(feats[:-1], slow=True)), m.bins)
        critic = critic - self.slow_reg * (slow * torch.log_softmax(critic_logits.float(), -1)).sum(-1)
        critic = (weights * critic).mean()
        metrics = {"imagined_return": returns[0].mean(), "actor_entropy": ents.mean().detach(), "value": value[0].mean(), "return_scale": scale.clone()}
        return actor + critic, metrics

    def loss(self, variables, batch, step: Step):
        g = torch.Generator().manual_seed((int(step.key) * 1000003 + int(step.step)) & 0x7FFFFFFF) if step.key is not None else None
        per, feat, hs, zs, wm_metrics = self.world_model_loss(batch, g)
        B, T = per.shape
        total = per.sum()
        mass = torch.tensor(float(B * T), device=per.device)
        behaviour, b_metrics = self.behaviour_loss(hs, zs, g)
        total = total + behaviour * mass
        metrics = {k: Ratio(v.detach() * mass, mass) for k, v in {**wm_metrics, **b_metrics}.items()}
        if self.imitation > 0 and "label" in batch:
            # a privileged teacher's actions at the student's own states (DAgger): the actor's mean is pulled to them
            out = self.model.actor(feat.detach())
            mean = out if self.model.discrete else torch.tanh(out.chunk(2, -1)[0])
            imit = ((mean - batch["label"].float()) ** 2).sum(-1)
            total = total + self.imitation * imit.sum()
            metrics["imitation"] = Ratio(imit.detach().sum(), mass)
        return Ratio(total, mass), Aux(metrics=metrics, effects={"slow_critic": True})

    def apply_effects(self, variables, effects) -> None:
        if effects.get("slow_critic"):
            with torch.no_grad():
                for s, p in zip(self.model.slow_critic.parameters(), self.model.critic.parameters()):
                    s.mul_(self.slow_decay).add_(p.detach(), alpha=1 - self.slow_decay)


# ------------------------------------------------------------------------------------------------ acting and collecting
class DreamerPolicy:
    """Acts in a ``Driven`` environment from the world model's filtered state; the memory is ``(h, z, previous action)``."""

    def __init__(self, model: DreamerModel, views_: Optional[Sequence[str]] = None, greedy: bool = False):
        self.model, self.views, self.greedy = model, views_, greedy

    def initial(self, n: int, device):
        h, z = self.model.rssm.initial(n, device)
        return h, z, torch.zeros(n, self.model.action_size, device=device)

    @torch.no_grad()
    def __call__(self, params, observation, memory, key):
        m = self.model
        obs = flat_observation(observation, self.views) if isinstance(observation, Mapping) else observation.float()
        n = obs.shape[0]
        if memory is None:
            memory = self.initial(n, obs.device)
        h, z, prev = memory
        first = observation["first"].bool() if isinstance(observation, Mapping) and "first" in observation else torch.zeros(n, dtype=torch.bool, device=obs.device)
        g = torch.Generator().manual_seed(int(key) & 0x7FFFFFFF)
        h, z, _, _ = m.rssm.obs_step(h, z, prev, m.encoder(D.symlog(obs)), first, g, mode=self.greedy)
        a, logp, _ = m.act(m.feat(h, z), g, self.greedy)
        return a, {"logp": logp}, (h, z, a)


class DreamerRollout:
    """Collects steps of a policy in a ``Driven`` environment into a replay of windows, each step stored as the objective reads it:
    the observation views, the action that led to it, the reward and the episode flags (and a teacher's label when the policy
    reports one)."""

    def __init__(self, env: Env, count: int, capacity: int = 1024, device="cpu"):
        self.env = env if isinstance(env, Driven) else Driven(env)
        self.count, self.replay = count, ReplayBuffer(capacity, count, device)
        self.carry: Optional[Carry] = None
        self.steps = 0

    def collect(self, policy, steps: int, key: int = 0) -> Dict[str, float]:
        if self.carry is None:
            self.carry = start(self.env, key, self.count)
        prev = getattr(self, "_prev_action", None)
        self.carry, tr = env_rollout(self.env, policy, None, self.carry, steps, reset=False)
        obs = tr.observation                                               # the step acted on: [steps, N, ...]
        for t in range(steps):
            acted = tr.action[t - 1] if t > 0 else (prev if prev is not None else torch.zeros_like(tr.action[0]))
            row = {k: v[t] for k, v in obs.items()}
            row["action"] = acted * (~row["first"].bool())[:, None].to(acted.dtype)
            if "label" in tr.extras:
                row["label"] = tr.extras["label"][t]
            self.replay.add(row)
        self._prev_action = tr.action[-1]
        self.steps += steps * self.count
        return {"reward": float(tr.step.observation["reward"].mean()), "episodes": float(tr.step.observation["last"].float().sum())}

    def sample(self, batch: int, length: int, generator=None) -> Dict[str, torch.Tensor]:
        return self.replay.sample(batch, length, generator)
