"""The named RL methods as compositions of this library's parts: an advantage estimator, a ratio and its clipping (the policy loss), a
reference penalty in the loss or in the reward, and a reduction - with DAPO's dynamic sampling and overlong punishment as batch steps.

| method | estimator | policy loss | clip (low, high) | reference penalty | reduction |
|---|---|---|---|---|---|
| grpo (arXiv 2402.03300) | group | ppo | 0.2, 0.2 | k3 in the loss, ``beta`` | sequence mean of token means |
| dapo (arXiv 2503.14476) | group | ppo | 0.2, 0.28 | none | token mean; varied groups only; overlong punishment |
| dr_grpo (arXiv 2503.20783) | group mean only | ppo | 0.2, 0.2 | none | token sums over a constant |
| gspo (arXiv 2507.18071) | group | sequence ratio | the run's | none | sequence mean of token means |
| cispo (arXiv 2506.13585) | group | clipped importance weight, stopped | none below, the run's above | none | token mean |
| gmpo (arXiv 2507.20673) | group | geometric mean of clipped ratios | e^-0.4, e^0.4 | none | sequence mean of token means |
| reinforce_pp (arXiv 2501.03262) | group baseline, batch scale | ppo | 0.2, 0.2 | k2 in the loss, ``beta`` | sequence mean of token means |
| rloo (arXiv 2402.14740) | leave-one-out | reinforce | none | k1 in the reward, ``reward_kl`` | token sums over a constant |

``method(name, model, group=...)`` builds the ``GRPO`` objective; a run may set only what the method leaves free (its group size, the
weight of its reference penalty where it has one, and the clip range where the paper tunes it).

Reference: src/dew/objectives/rl/methods.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

import torch

from .policy import GRPO


@dataclass(frozen=True)
class Method:
    name: str
    advantage: str
    rule: str
    clip: Optional[Tuple[float, float]]           # None: the run's
    kl_kind: Optional[str] = None                 # a reference penalty in the loss
    beta: float = 0.0
    reward_kl: float = 0.0                        # a k1 reference penalty folded into the reward
    reduction: str = "seq-mean-token-mean"
    varied_groups: bool = False                   # DAPO: groups whose rewards are all alike carry no signal and are dropped
    overlong: bool = False                        # DAPO: soft punishment of completions near the length limit
    free: Tuple[str, ...] = ("group",)


METHODS: Dict[str, Method] = {m.name: m for m in (
    Method("grpo", "grpo", "ppo", (0.2, 0.2), kl_kind="k3", beta=0.04, free=("group", "beta")),
    Method("dapo", "grpo", "ppo", (0.2, 0.28), reduction="token-mean", varied_groups=True, overlong=True),
    Method("dr_grpo", "dr_grpo", "ppo", (0.2, 0.2), reduction="seq-mean-token-sum-norm"),
    Method("gspo", "grpo", "gspo", None, free=("group", "clip", "clip_high")),
    Method("cispo", "grpo", "cispo", None, reduction="token-mean", free=("group", "clip_high")),
    Method("gmpo", "grpo", "gmpo", (0.4, 0.4)),
    Method("reinforce_pp", "global", "ppo", (0.2, 0.2), kl_kind="k2", beta=0.01, free=("group", "beta")),
    Method("rloo", "rloo", "reinforce", None, reward_kl=0.01, reduction="seq-mean-token-sum-norm", free=("group", "reward_kl")),
)}


def method(name: str, model, group: int = 8, **free: Any) -> GRPO:
    if name not in METHODS:
        raise KeyError(f"RL method {name!r}; known: {sorted(METHODS)}")
    m = METHODS[name]
    extra = sorted(set(free) - set(m.free))
    if extra:
        raise ValueError(f"{name} fixes {extra}; a run may set only {list(m.free)}")
    if m.clip is None:
        low = free.get("clip", 3e-4 if name == "gspo" else 1.0)
        high = free.get("clip_high", 4e-4 if name == "gspo" else 0.28 if name == "cispo" else low)
    else:
        low, high = m.clip
    obj = GRPO(model, group=group, clip=low, clip_high=high, kl=float(free.get("beta", m.beta)) if m.kl_kind else 0.0, kl_kind=m.kl_kind or "k3",
               rule=m.rule, advantage=m.advantage, reduction=m.reduction)
    obj.method = m
    obj.reward_kl = float(free.get("reward_kl", m.reward_kl))
    return obj


# ------------------------------------------------------------------------------------------------ batch steps
def varied_groups(batch: Mapping[str, torch.Tensor], group: int) -> Tuple[Dict[str, torch.Tensor], float]:
    """DAPO's dynamic sampling, the filtering half: the rows of groups whose rewards differ, and the share of groups kept.  (The sampling
    half - drawing more prompts until the batch is full - is the collector's: it calls this and keeps drawing.)"""
    r = batch["rewards"].reshape(-1, group)
    keep = (r.max(1).values - r.min(1).values) > 0
    rows = keep[:, None].expand(-1, group).reshape(-1)
    return {k: (v[rows] if torch.is_tensor(v) and v.shape[:1] == rows.shape else v) for k, v in batch.items()}, float(keep.float().mean())


def overlong_punishment(lengths: torch.Tensor, limit: int, buffer: int) -> torch.Tensor:
    """DAPO's soft punishment: nothing up to ``limit - buffer`` tokens, falling linearly to -1 at ``limit``, -1 beyond."""
    over = (lengths.float() - (limit - buffer)) / max(1, buffer)
    return -over.clamp(0.0, 1.0)


def reward_with_reference(rewards: torch.Tensor, logp: torch.Tensor, ref_logp: torch.Tensor, mask: torch.Tensor, weight: float) -> torch.Tensor:
    """RLOO's reference penalty: the sequence's summed k1 estimate ``log pi - log pi_ref`` over its completion, times ``weight``, off the reward."""
    return rewards - weight * ((logp.float() - ref_logp.float()) * mask.float()).sum(-1)


def prepare(obj: GRPO, batch: Mapping[str, torch.Tensor], limit: Optional[int] = None, buffer: int = 0, ref_logprobs: Optional[torch.Tensor] = None
            ) -> Tuple[Dict[str, torch.Tensor], Dict[str, float]]:
    """What a method does to a collected batch before the loss reads it; returns the batch and what it did, for the log."""
    m: Method = obj.method
    out, report = dict(batch), {}
    mask = out["mask"][:, 1:].float()
    if m.overlong and limit:
        pen = overlong_punishment(mask.sum(-1), limit, buffer)
        out["rewards"] = out["rewards"].float() + pen.to(out["rewards"].device)
        report["overlong_share"] = float((pen < 0).float().mean())
    if obj.reward_kl and ref_logprobs is not None:
        out["rewards"] = reward_with_reference(out["rewards"].float(), out["old_logprobs"], ref_logprobs, mask, obj.reward_kl)
    if m.varied_groups:
        out, kept = varied_groups(out, obj.group)
        report["groups_kept"] = kept
    return out, report
