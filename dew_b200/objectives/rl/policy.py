"""Policy-gradient objectives over sampled completions, assembled from ``dew_b200.rl.advantage`` and ``dew_b200.rl.surrogate``.

``GRPO``  group-relative advantages (``advantage='grpo' | 'dr_grpo' | 'rloo'``) under one of the update rules ``rule='ppo'`` (clipped
          ratio with asymmetric clips and the dual clip), ``'gspo'`` (sequence-level ratio), ``'cispo'``, ``'gmpo'`` or ``'reinforce'``;
          a KL pull to the reference kept in the EMA slot (``kl_kind`` k1 / abs / k2 / k3); corrections for a sampler whose
          log-probabilities differ from the trainer's (``behavior_logprobs`` in the batch: truncated importance weights, IcePop's
          band, sequence rejection); any of ``surrogate.aggregate``'s reductions
``PPO``   clipped surrogate + clipped value loss + entropy bonus; advantages given, or computed from token rewards and old values
          by masked GAE with whitening

Reference: src/dew/objectives/rl (GRPO, PPO and their options), src/dew/rl/advantage.py, src/dew/rl/surrogate.py."""
from __future__ import annotations

from typing import Optional

import torch

from ...rl import advantage as A
from ...rl import surrogate as S
from ..base import Aux, EMASpec, Objective, Ratio, Step


def group_advantages(rewards: torch.Tensor, group: int, eps: float = 1e-6) -> torch.Tensor:
    """Standardise rewards within each group of ``group`` completions of the same prompt."""
    return A.group_advantage(rewards.float(), group, eps)


def gae(rewards, values, dones, gamma: float = 0.99, lam: float = 0.95):
    """Generalised advantage estimation over ``[T, B]`` trajectories; ``values`` has one extra bootstrap row."""
    return A.generalized_advantages(rewards, values[:-1], dones, gamma, lam, bootstrap=values[-1])


def _token_logprobs(logits, tokens):
    return torch.log_softmax(logits.float(), -1).gather(-1, tokens[:, 1:, None]).squeeze(-1)


def forked_logits(call, tokens: torch.Tensor, full_mask: torch.Tensor, window: int, min_prefix: int = 8) -> torch.Tensor:
    """Logits ``[B, S-1, V]`` of the inputs ``tokens[:, :-1]`` computed with rows that begin alike laid out once (``data.forked_rows``):
    each row is cut after its last masked token, the rows are grouped by common prefix and packed, ``call(tokens, positions=...,
    segment_ids=forks)`` runs the model, and the outputs are gathered back row by row.  Places past a row's last masked token hold zeros,
    which the mask never reads.  (The grouping reads the token ids on the host.)"""
    from ...data.forked_rows import ForkedRows
    B, S = tokens.shape
    last = torch.where(full_mask.bool().any(1), S - full_mask.bool().flip(1).float().argmax(1), torch.full((B,), S, device=tokens.device))
    rows = [tokens[i, :max(1, int(n) - 1)].tolist() for i, n in enumerate(last.tolist())]
    packed = ForkedRows.pack(rows, window=window, min_prefix=min_prefix)
    dev = tokens.device
    out = call(packed.tokens.to(dev), positions=packed.positions.to(dev), segment_ids=packed.forks.to(dev))
    out = out[0] if isinstance(out, tuple) else out
    padded, _ = packed.padded(out)
    return torch.nn.functional.pad(padded, (0, 0, 0, S - 1 - padded.shape[1]))


_ADVANTAGES = {"grpo": lambda r, g: A.group_advantage(r, g), "dr_grpo": A.dr_grpo_advantage, "rloo": A.rloo_advantage, "global": A.global_advantage}
RULES = ("ppo", "gspo", "cispo", "gmpo", "reinforce")


class GRPO(Objective):
    starts_from_model = True
    """batch: ``tokens [B,S]``, ``mask [B,S]`` (1 on completion tokens), ``rewards [B]``, ``old_logprobs [B,S-1]``; optionally
    ``behavior_logprobs [B,S-1]`` (what the sampling engine reported) and ``advantages [B]`` (overrides the group estimate)."""

    def __init__(self, model, group: int = 4, clip: float = 0.2, kl: float = 0.04, *, clip_high: Optional[float] = None,
                 dual_clip: Optional[float] = None, rule: str = "ppo", advantage: str = "grpo", reduction: Optional[str] = None,
                 kl_kind: str = "k3", importance: Optional[str] = None, importance_threshold: float = 2.0, band=(0.5, 2.0),
                 share_prefix: bool = False, min_prefix: int = 8):
        # share_prefix: a group's rows begin with the same prompt; lay the prompt out once per group (data.forked_rows) instead of once per row
        self.share_prefix, self.min_prefix = share_prefix, min_prefix
        if rule not in RULES:
            raise ValueError(f"unknown update rule {rule!r}; known: {RULES}")
        if advantage not in _ADVANTAGES:
            raise ValueError(f"unknown advantage estimator {advantage!r}; known: {sorted(_ADVANTAGES)}")
        if importance not in (None, "truncated", "band", "reject"):
            raise ValueError("importance is None, 'truncated' (TIS), 'band' (IcePop) or 'reject' (sequence rejection)")
        self.model, self.group, self.clip, self.kl = model, group, clip, kl
        self.clip_high, self.dual_clip, self.rule, self.advantage = clip_high, dual_clip, rule, advantage
        self.reduction = reduction or {"gspo": "seq-mean-token-mean", "gmpo": "seq-mean-token-mean", "dr_grpo": "seq-mean-token-sum-norm"}.get(
            rule if rule in ("gspo", "gmpo") else advantage, "token-mean")
        self.kl_kind, self.importance, self.importance_threshold, self.band = kl_kind, importance, importance_threshold, band
        self.ema_decay = EMASpec.constant(1.0)

    def _logits(self, variables, tokens, full_mask):
        """Logits ``[B, S-1, V]`` of the inputs ``tokens[:, :-1]``; with ``share_prefix`` through the forked layout."""
        if not self.share_prefix:
            return self.apply(variables, tokens[:, :-1])
        S = tokens.shape[1]
        return forked_logits(lambda *a, **k: self.apply(variables, *a, **k), tokens, full_mask, max(S - 1, self.group * (S - 1) // 2), self.min_prefix)

    def loss(self, variables, batch, step: Step):
        tokens, mask = batch["tokens"], batch["mask"][:, 1:].bool()
        lp = _token_logprobs(self._logits(variables, tokens, batch["mask"]), tokens)
        old = batch["old_logprobs"].float()
        adv = batch["advantages"].float() if "advantages" in batch else _ADVANTAGES[self.advantage](batch["rewards"].float(), self.group)
        adv = adv.to(lp.device)[:, None].expand_as(lp)
        metrics = {}
        if self.rule == "ppo":
            terms, m = S.clipped_surrogate_terms(S.token_log_ratio(lp, old), adv, mask, self.clip, self.clip_high, self.dual_clip)
        elif self.rule == "gspo":
            terms, m = S.clipped_surrogate_terms(S.sequence_log_ratio(lp, old, mask), adv, mask, self.clip, self.clip_high, None)
        elif self.rule == "cispo":
            terms, m = S.cispo_terms(lp, old, adv, mask, self.clip, self.clip if self.clip_high is None else self.clip_high)
        elif self.rule == "gmpo":
            terms, m = S.gmpo_terms(lp, old, adv, mask, self.clip, self.clip if self.clip_high is None else self.clip_high)
        else:
            terms, m = S.reinforce_terms(lp, adv), {}
        keep = mask
        if self.importance is not None and "behavior_logprobs" in batch:
            beh = batch["behavior_logprobs"].float()
            if self.importance == "truncated":
                terms = terms * S.behavior_importance_weights(old, beh, mask, self.importance_threshold)
            elif self.importance == "band":
                terms = terms * S.behavior_band_weights(old, beh, mask, *self.band)
            else:
                keep = S.sequence_rejection_mask(old, beh, mask, *self.band).bool()
            metrics.update({f"mismatch_{k}": Ratio(v.detach(), torch.tensor(1.0)) for k, v in S.mismatch_metrics(old, beh, mask).items()})
        if self.kl and step.ema is not None:
            with torch.no_grad():
                ref = _token_logprobs(self.apply(step.ema, tokens[:, :-1]), tokens)
            klv = S.kl_penalty(lp, ref, self.kl_kind)
            terms = terms + self.kl * klv
            metrics["kl"] = Ratio((klv.detach() * mask).sum(), mask.sum())
        count = mask.float().sum()
        for k, v in m.items():
            metrics[k] = Ratio(v.detach() * count, count)
        if self.reduction == "token-mean":
            kept = keep.float()
            return Ratio((torch.where(keep, terms, torch.zeros_like(terms))).sum(), kept.sum().clamp_min(1)), Aux(metrics=metrics)
        rows = (keep.float().sum(-1) > 0).float().sum().clamp_min(1)
        return Ratio(S.aggregate(terms, keep, self.reduction) * rows, rows), Aux(metrics=metrics)


class PPO(Objective):
    starts_from_model = True
    """The model returns ``(logits, values)``; batch: ``tokens, mask, old_logprobs`` and either ``advantages [B,S-1]`` + ``returns
    [B,S-1]`` or ``token_rewards [B,S-1]`` + ``old_values [B,S-1]`` (masked GAE with whitening computes the former from the latter)."""

    def __init__(self, model, clip: float = 0.2, value_coef: float = 0.5, entropy_coef: float = 0.0, *, clip_high: Optional[float] = None,
                 dual_clip: Optional[float] = None, value_clip: Optional[float] = None, gamma: float = 1.0, lam: float = 0.95):
        self.model, self.clip, self.value_coef, self.entropy_coef = model, clip, value_coef, entropy_coef
        self.clip_high, self.dual_clip, self.value_clip, self.gamma, self.lam = clip_high, dual_clip, value_clip, gamma, lam

    def loss(self, variables, batch, step: Step):
        tokens, maskb = batch["tokens"], batch["mask"][:, 1:].bool()
        mask = maskb.float()
        logits, values = self.apply(variables, tokens[:, :-1])
        values = values.float().squeeze(-1)
        lp = _token_logprobs(logits, tokens)
        if "advantages" in batch:
            adv, returns = batch["advantages"].float(), batch["returns"].float()
        else:
            adv, returns = A.gae(batch["token_rewards"].float(), batch["old_values"].float(), maskb, self.gamma, self.lam)
        policy, pm = S.clipped_surrogate_terms(S.token_log_ratio(lp, batch["old_logprobs"].float()), adv, maskb, self.clip, self.clip_high, self.dual_clip)
        if self.value_clip is not None and "old_values" in batch:
            value, _ = S.clipped_value_loss_terms(values, batch["old_values"].float(), returns, self.value_clip)
        else:
            value = 0.5 * (values - returns) ** 2
        p = torch.softmax(logits.float(), -1)
        ent = -(p * torch.log(p.clamp_min(1e-12))).sum(-1)
        per = policy + self.value_coef * value - self.entropy_coef * ent
        m = mask.sum()
        return Ratio((per * mask).sum(), m), Aux(metrics={"entropy": Ratio((ent.detach() * mask).sum(), m),
                                                           "value_loss": Ratio((value.detach() * mask).sum(), m),
                                                           "clip_fraction": Ratio(pm["clip_fraction"].detach() * m, m)})


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
