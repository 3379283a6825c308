"""Update rules: plain functions from log-probabilities and advantages to per-token loss terms, their reductions and metrics.

Everything takes ``[B, T]`` tensors and a response mask; nothing here runs a model.  Conventions: ``log_ratio`` is
``log pi(a) - log pi_old(a)`` clamped to +-20; terms are *losses* (to minimise); reductions are ``aggregate``'s modes.

``clipped_surrogate_terms``  PPO / GRPO: ``max(-A r, -A clip(r, 1 - lo, 1 + hi))`` with the dual clip for negative advantages
``sequence_log_ratio``       GSPO: the sequence ratio is the geometric mean of the token ratios, its gradient per token
``cispo_terms``              CISPO: ``-sg(clip(r)) A log pi``
``gmpo_terms``               GMPO: the geometric mean of a sequence's clipped token ratios, signed by its advantage
``reinforce_terms``          ``-A log pi`` (RLOO's estimator)
``k3_kl`` / ``sampled_kl``   Schulman's k3 estimate ``exp(d) - d - 1``
``clipped_value_loss_terms`` PPO's clipped value loss
``behavior_importance_weights`` / ``behavior_band_weights`` / ``sequence_rejection_mask`` / ``mismatch_metrics``
                             corrections and diagnostics for a sampler (an inference engine) whose log-probabilities differ
                             from the trainer's: truncated importance weights, IcePop's band, sequence-level rejection
``preference_logsigmoid_terms``  DPO's sigmoid loss with label smoothing, and the implied rewards

Reference: src/dew/rl/surrogate.py (the same function names).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from .advantage import MEAN_EPS, masked_mean

LOG_RATIO_CLAMP = 20.0


def token_log_ratio(logp: torch.Tensor, old_logp: torch.Tensor) -> torch.Tensor:
    return (logp.float() - old_logp.float()).clamp(-LOG_RATIO_CLAMP, LOG_RATIO_CLAMP)


def segment_mean(x: torch.Tensor, mask: torch.Tensor, segments: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Each position's masked mean over its sequence, broadcast back to ``[B, T]``.  A sequence is a row, or with ``segments``
    (packed rows) one run of equal non-zero ids within a row."""
    m = mask.to(x.dtype)
    kept = torch.where(mask.bool(), x, torch.zeros_like(x))
    if segments is None:
        return (kept.sum(-1, keepdim=True) / m.sum(-1, keepdim=True).clamp_min(1)).expand_as(x)
    B, T = x.shape
    S = int(segments.max()) + 1
    idx = segments.long()
    total = torch.zeros(B, S, dtype=x.dtype, device=x.device).scatter_add(1, idx, kept)
    count = torch.zeros(B, S, dtype=x.dtype, device=x.device).scatter_add(1, idx, m)
    return (total / count.clamp_min(1)).gather(1, idx)


def aggregate(terms: torch.Tensor, mask: torch.Tensor, mode: str = "token-mean", segments: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Reduce per-token terms to a scalar: ``token-mean`` (all kept tokens weigh the same), ``seq-mean-token-sum`` (sum inside a
    sequence, mean over sequences), ``seq-mean-token-mean`` (mean inside, mean over), ``seq-mean-token-sum-norm`` (sum inside,
    over the row length, mean over sequences: Dr. GRPO's constant normaliser)."""
    m = mask.to(terms.dtype)
    if mode == "token-mean":
        return masked_mean(terms, mask)
    if segments is not None:
        raise ValueError("sequence-level reductions of packed rows: unpack first, or use token-mean")
    sums = torch.where(mask.bool(), terms, torch.zeros_like(terms)).sum(-1)
    live = (m.sum(-1) > 0).to(terms.dtype)
    n = live.sum().clamp_min(1)
    if mode == "seq-mean-token-sum":
        return (sums * live).sum() / n
    if mode == "seq-mean-token-mean":
        return (sums / m.sum(-1).clamp_min(1) * live).sum() / n
    if mode == "seq-mean-token-sum-norm":
        return (sums / terms.shape[-1] * live).sum() / n
    raise ValueError(f"unknown reduction {mode!r}")


def sequence_log_ratio(logp: torch.Tensor, old_logp: torch.Tensor, mask: torch.Tensor, segments=None) -> torch.Tensor:
    """GSPO's sequence-level log ratio with a per-token gradient: the value at every token of a sequence is the sequence's mean
    token log ratio, and its gradient flows through that token's own log-probability (``logp - sg(logp) + sg(mean)``)."""
    seq = segment_mean(token_log_ratio(logp, old_logp), mask, segments)
    return (logp.float() - logp.float().detach() + seq.detach()).clamp(max=10.0)


def clipped_surrogate_terms(log_ratio: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor, clip_low: float = 0.2,
                            clip_high: Optional[float] = None, dual_clip: Optional[float] = 3.0) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    clip_high = clip_low if clip_high is None else clip_high
    if dual_clip is not None and dual_clip <= 1.0:
        raise ValueError("the dual clip bounds the ratio for negative advantages from above: it must exceed 1")
    A = advantages.float()
    ratio = log_ratio.exp()
    plain = -A * ratio
    clipped = -A * ratio.clamp(1 - clip_low, 1 + clip_high)
    upper = torch.maximum(plain, clipped)
    metrics = {"clip_fraction": masked_mean((clipped > plain).float(), mask), "approx_kl": masked_mean(-log_ratio, mask)}
    if dual_clip is None:
        return upper, metrics
    floor = -A * dual_clip
    lower = torch.minimum(floor, upper)
    metrics["dual_clip_fraction"] = masked_mean(((upper > floor) & (A < 0)).float(), mask)
    return torch.where(A < 0, lower, upper), metrics


def cispo_terms(logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor, clip_low: float = 1.0,
                clip_high: float = 0.28) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    log_ratio = token_log_ratio(logp, old_logp)
    ratio = log_ratio.exp()
    held = ratio.clamp(1 - clip_low, 1 + clip_high).detach()
    terms = -held * advantages.float() * logp.float()
    return terms, {"clip_fraction": masked_mean((held != ratio.detach()).float(), mask), "approx_kl": masked_mean(-log_ratio, mask)}


def gmpo_terms(logp, old_logp, advantages, mask, clip_low: float = 0.4, clip_high: float = 0.4):
    """Each sequence's term ``-A exp(mean_t log m_t)``, ``m_t`` the token ratio clipped in log space on the side that would
    otherwise grow the objective, given to each of its tokens (so ``aggregate(..., 'seq-mean-token-mean')`` recovers the
    sequence mean)."""
    d = logp.float() - old_logp.float()
    sign = torch.sign(advantages.float())
    held = sign * torch.minimum(sign * d, sign * d.clamp(-clip_low, clip_high))
    m = mask.to(d.dtype)
    seq = (held * m).sum(-1) / (m.sum(-1) + MEAN_EPS)
    adv = (advantages.float() * m).sum(-1) / (m.sum(-1) + MEAN_EPS)
    terms = (-adv * seq.exp())[:, None].expand_as(d)
    return terms, {"clip_fraction": masked_mean((held != d).float(), mask), "approx_kl": masked_mean(-d, mask)}


def reinforce_terms(logp: torch.Tensor, advantages: torch.Tensor) -> torch.Tensor:
    return -advantages.float() * logp.float()


def k3_kl(logp: torch.Tensor, ref_logp: torch.Tensor) -> torch.Tensor:
    """Per-token estimate of KL(pi || pi_ref): ``exp(d) - d - 1`` with ``d = log pi_ref - log pi``, clamped to [-10, 10]."""
    d = (ref_logp.float() - logp.float()).clamp(-LOG_RATIO_CLAMP, LOG_RATIO_CLAMP)
    return sampled_kl(d).clamp(-10.0, 10.0)


def sampled_kl(r: torch.Tensor) -> torch.Tensor:
    """``exp(r) - r - 1`` as ``expm1(r) - r``: for small ``r`` the terms the estimate is made of survive the rounding."""
    return torch.expm1(r) - r


def kl_penalty(logp, ref_logp, kind: str = "k3") -> torch.Tensor:
    d = logp.float() - ref_logp.float()
    if kind == "k1":
        return d
    if kind == "abs":
        return d.abs()
    if kind == "k2":
        return 0.5 * d * d
    if kind == "k3":
        return k3_kl(logp, ref_logp)
    raise ValueError(f"unknown KL estimate {kind!r}; known: k1, abs, k2, k3")


def clipped_value_loss_terms(values: torch.Tensor, old_values: torch.Tensor, returns: torch.Tensor, clip: float = 0.5):
    held = torch.maximum(torch.minimum(values, old_values + clip), old_values - clip)
    plain, clipped = (values - returns) ** 2, (held - returns) ** 2
    return 0.5 * torch.maximum(plain, clipped), (clipped > plain).float()


# ------------------------------------------------------------------------------------------------ sampler / trainer mismatch
def behavior_importance_weights(proximal_logp, behavior_logp, mask, threshold: float = 2.0) -> torch.Tensor:
    """Truncated importance sampling: ``min(exp(log pi_prox - log pi_behaviour), threshold)`` per token, detached, zero outside
    the mask.  ``proximal`` is the trainer's recomputation under the sampling weights, ``behaviour`` what the engine reported."""
    w = (proximal_logp.float() - behavior_logp.float()).clamp(-LOG_RATIO_CLAMP, LOG_RATIO_CLAMP).exp().clamp(max=threshold)
    return (w * mask.to(w.dtype)).detach()


def behavior_band_weights(proximal_logp, behavior_logp, mask, low: float = 0.5, high: float = 2.0) -> torch.Tensor:
    """IcePop: the token ratio inside ``[low, high]``, zero outside."""
    w = (proximal_logp.float() - behavior_logp.float()).clamp(-LOG_RATIO_CLAMP, LOG_RATIO_CLAMP).exp()
    return (torch.where((w >= low) & (w <= high), w, torch.zeros_like(w)) * mask.to(w.dtype)).detach()


def sequence_rejection_mask(proximal_logp, behavior_logp, mask, low: float = 0.5, high: float = 2.0, geometric: bool = True) -> torch.Tensor:
    """1 for every token of a sequence whose log-ratio statistic (its mean with ``geometric``, else its sum) lies in
    ``[log low, log high]``, 0 for every token of the others."""
    d = (proximal_logp.float() - behavior_logp.float()) * mask.to(torch.float32)
    stat = d.sum(-1) / mask.sum(-1).clamp_min(1) if geometric else d.sum(-1)
    keep = (stat >= math.log(low)) & (stat <= math.log(high))
    return keep[:, None].to(torch.float32) * mask.to(torch.float32)


def mismatch_metrics(proximal_logp, behavior_logp, mask) -> Dict[str, torch.Tensor]:
    d = proximal_logp.float() - behavior_logp.float()
    r = d.exp()
    return {"kl": masked_mean(-d, mask), "k3_kl": masked_mean(r - d - 1, mask), "ratio_mean": masked_mean(r, mask),
            "ratio_max": torch.where(mask.bool(), r, torch.zeros_like(r)).max(), "ppl_gap": masked_mean(d.abs(), mask)}


# ------------------------------------------------------------------------------------------------ preferences
def preference_logsigmoid_terms(chosen_logp, rejected_logp, ref_chosen_logp, ref_rejected_logp, chosen_mask, rejected_mask,
                                beta: float = 0.1, label_smoothing: float = 0.0):
    """DPO: each completion's log-ratio is the masked sum of its policy log-probabilities minus the reference's; the loss is
    ``-(1 - s) logsigmoid(beta (dc - dr)) - s logsigmoid(-beta (dc - dr))``.  Returns (terms [B], chosen rewards, rejected rewards)."""
    dc = ((chosen_logp.float() - ref_chosen_logp.float()) * chosen_mask.to(torch.float32)).sum(-1)
    dr = ((rejected_logp.float() - ref_rejected_logp.float()) * rejected_mask.to(torch.float32)).sum(-1)
    z = beta * (dc - dr)
    terms = -(1 - label_smoothing) * F.logsigmoid(z) - label_smoothing * F.logsigmoid(-z)
    return terms, (beta * dc).detach(), (beta * dr).detach()
