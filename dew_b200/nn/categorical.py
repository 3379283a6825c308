"""The categorical distribution over a class axis (the last): log-probabilities, cross entropies, divergences, proper scoring
rules, and the block-wise log partition a chunked head combines.

Everything computes in float32 at least (float64 stays float64): a bf16 log partition over a large vocabulary puts bf16's
8-bit mantissa into every score.  ``where`` (a bool mask over the classes, broadcastable to the logits) leaves classes out:
they take no probability and add no term to any sum.

Reference: src/dew/nn/categorical.py (``log_probs``, ``cross_entropy``, ``soft_cross_entropy``, ``kl_divergence``, ``entropy``,
``brier``, ``spherical``, ``ranked_probability``, ``smoothed``, ``group_divergence``, ``rescaled``, ``target_loss``,
``segment_log_partition``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def _wide(x: torch.Tensor) -> torch.Tensor:
    return x if x.dtype == torch.float64 else x.float()


def _masked(logits: torch.Tensor, where: Optional[torch.Tensor]) -> torch.Tensor:
    logits = _wide(logits)
    return logits if where is None else logits.masked_fill(~where, float("-inf"))


def log_probs(logits: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    return torch.log_softmax(_masked(logits, where), -1)


def probs(logits: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    return torch.softmax(_masked(logits, where), -1)


def _dot(p: torch.Tensor, logp: torch.Tensor) -> torch.Tensor:
    """sum_c p_c logp_c with 0 * (-inf) = 0 (a class of no probability adds nothing)."""
    return torch.where(p > 0, p * logp.clamp_min(torch.finfo(logp.dtype).min), torch.zeros_like(logp)).sum(-1)


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    """-log p(label) per row."""
    return -log_probs(logits, where).gather(-1, labels[..., None]).squeeze(-1)


def soft_cross_entropy(logits: torch.Tensor, target: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    return -_dot(_wide(target), log_probs(logits, where))


def entropy(logits: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    lp = log_probs(logits, where)
    return -_dot(lp.exp(), lp)


def kl_divergence(logits: torch.Tensor, reference_logits: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    """KL(p || q) with p from ``logits`` and q from ``reference_logits``."""
    lp, lq = log_probs(logits, where), log_probs(reference_logits, where)
    p = lp.exp()
    return torch.where(p > 0, p * (lp - lq.clamp_min(torch.finfo(lq.dtype).min)), torch.zeros_like(p)).sum(-1)


def smoothed(target: torch.Tensor, amount: float, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``(1 - amount) target + amount * even`` over the classes a row holds."""
    target = _wide(target)
    if where is None:
        even = torch.full_like(target, 1.0 / target.shape[-1])
    else:
        w = where.expand_as(target).to(target.dtype)
        even = w / w.sum(-1, keepdim=True).clamp_min(1)
    return (1 - amount) * target + amount * even


def brier(logits: torch.Tensor, target: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The quadratic score's charge: sum_c (p_c - t_c)^2."""
    return ((probs(logits, where) - _wide(target)) ** 2).sum(-1)


def spherical(logits: torch.Tensor, target: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The spherical score's charge: 1 - <p, t> / |p|."""
    p = probs(logits, where)
    return 1 - (p * _wide(target)).sum(-1) / p.norm(dim=-1).clamp_min(1e-30)


def ranked_probability(logits: torch.Tensor, target: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The ranked probability score over ordered classes: sum_c (CDF_p(c) - CDF_t(c))^2."""
    return ((probs(logits, where).cumsum(-1) - _wide(target).cumsum(-1))[..., :-1] ** 2).sum(-1)


def group_divergence(logits: torch.Tensor, where: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Mean over the members of a group ``[..., members, classes]`` of KL(member || the group's mean distribution): the
    generalised Jensen-Shannon divergence among the members."""
    p = probs(logits, where)
    mean = p.mean(-2, keepdim=True)
    term = torch.where(p > 0, p * (torch.log(p.clamp_min(1e-38)) - torch.log(mean.clamp_min(1e-38))), torch.zeros_like(p))
    return term.sum(-1).mean(-1)


# ---------------------------------------------------------------------------------------------- block-wise partition
def rescaled(running: Optional[Tuple[torch.Tensor, torch.Tensor]], block_logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Combine a running ``(max, sum of exp(logit - max))`` per row with another block of the vocabulary."""
    block = _wide(block_logits)
    bmax = block.amax(-1)
    if running is None:
        return bmax, torch.exp(block - bmax[..., None]).sum(-1)
    m, s = running
    new = torch.maximum(m, bmax)
    return new, s * torch.exp(m - new) + torch.exp(block - new[..., None]).sum(-1)


def log_partition(running: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    m, s = running
    return m + torch.log(s)


def target_loss(running: Tuple[torch.Tensor, torch.Tensor], target_logit: torch.Tensor) -> torch.Tensor:
    """A label's cross entropy from the combined partition and the label's own logit."""
    return log_partition(running) - _wide(target_logit)


def segment_log_partition(logits: torch.Tensor, segments: torch.Tensor, count: int) -> torch.Tensor:
    """Log partition of each segment of a ragged row: ``logits [n]``, ``segments [n]`` (ids in ``[0, count)``) -> ``[count]``
    (``-inf`` for an empty segment)."""
    x = _wide(logits)
    m = torch.full((count,), float("-inf"), dtype=x.dtype, device=x.device).scatter_reduce(0, segments, x, "amax", include_self=True)
    safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    s = torch.zeros(count, dtype=x.dtype, device=x.device).index_add_(0, segments, torch.exp(x - safe[segments]))
    return torch.where(s > 0, safe + torch.log(s.clamp_min(1e-38)), torch.full_like(s, float("-inf")))
