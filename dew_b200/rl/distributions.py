"""DreamerV3's output transforms and distributions on plain tensors (arXiv 2301.04104).

``symlog`` compresses a target's magnitude and ``symexp`` inverts it.  A two-hot distribution over the bins
``symexp(linspace(-20, 20, 255))`` predicts a scalar of any scale as its bins' expectation - summed from both ends toward the
middle so uniform probabilities predict exactly zero - and is trained by the cross-entropy against the target's two-hot
encoding (its weight split between the two neighbouring bins).  A categorical latent mixes its softmax with 1 % uniform
(``unimix``) and is drawn one-hot with the gradient of its probabilities (straight through).  A continuous policy's normal reads
its per-coordinate terms here, a tanh-squashed one its log-Jacobian too.

Reference: src/dew/rl/distributions.py (``symlog``, ``symexp``, ``twohot_bins``, ``twohot_mean``, ``twohot_loss``,
``unimix_log_probs``, ``normal_log_density``, ``normal_entropy``, ``tanh_log_jacobian``, ``onehot_sample``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def symlog(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.log1p(x.abs())


def symexp(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.expm1(x.abs())


def twohot_bins(count: int = 255, limit: float = 20.0, device=None, dtype=torch.float32) -> torch.Tensor:
    """``symexp`` of ``count`` points evenly spaced over ``[-limit, limit]``, the negative half mirrored from the positive one so
    the bins are exactly symmetric."""
    if count % 2 == 1:
        half = symexp(torch.linspace(-limit, 0.0, (count - 1) // 2 + 1, dtype=torch.float64))
        bins = torch.cat([half, -half[:-1].flip(0)])
    else:
        half = symexp(torch.linspace(-limit, -limit / (count - 1), count // 2, dtype=torch.float64))     # no bin at zero
        bins = torch.cat([half, -half.flip(0)])
    return bins.to(device=device, dtype=dtype)


def twohot_mean(logits: torch.Tensor, bins: torch.Tensor) -> torch.Tensor:
    """The expectation of ``bins`` under ``softmax(logits)``, summed outward-in from both ends to the middle bin, so symmetric
    bins under uniform probabilities give exactly zero."""
    p = torch.softmax(logits.float(), -1)
    n = bins.shape[0]
    if n % 2 == 1:
        m = (n - 1) // 2
        left = (p[..., :m] * bins[:m]).sum(-1)
        right = (p[..., m + 1:] * bins[m + 1:]).flip(-1).sum(-1)
        return left + right + p[..., m] * bins[m]
    m = n // 2
    return (p[..., :m] * bins[:m]).sum(-1) + (p[..., m:] * bins[m:]).flip(-1).sum(-1)


def twohot(target: torch.Tensor, bins: torch.Tensor) -> torch.Tensor:
    """The two-hot encoding ``[..., bins]`` of ``target``: weight on the bins either side of it, each in proportion to the
    other's distance; all of it on the first or last bin past the ends."""
    t = target.float()
    n = bins.shape[0]
    below = (torch.searchsorted(bins, t.contiguous(), right=True) - 1).clamp(0, n - 1)
    above = (below + 1).clamp(0, n - 1)
    lo, hi = bins[below], bins[above]
    same = above == below
    d_lo, d_hi = (t - lo).abs(), (hi - t).abs()
    total = (d_lo + d_hi).clamp_min(1e-30)
    w_lo = torch.where(same, torch.ones_like(t), d_hi / total)
    w_hi = torch.where(same, torch.zeros_like(t), d_lo / total)
    past = (t <= bins[0]) | (t >= bins[-1])
    w_lo = torch.where(past & (t <= bins[0]), torch.ones_like(t), w_lo)
    w_hi = torch.where(past & (t <= bins[0]), torch.zeros_like(t), w_hi)
    return F.one_hot(below, n).to(t.dtype) * w_lo[..., None] + F.one_hot(above, n).to(t.dtype) * w_hi[..., None]


def twohot_loss(logits: torch.Tensor, target: torch.Tensor, bins: torch.Tensor) -> torch.Tensor:
    return -(twohot(target, bins) * torch.log_softmax(logits.float(), -1)).sum(-1)


def unimix_log_probs(logits: torch.Tensor, unimix: float = 0.01) -> torch.Tensor:
    """Log-probabilities of ``(1 - unimix) softmax(logits) + unimix / n``, finite wherever the logits are."""
    lp = torch.log_softmax(logits.float(), -1)
    if unimix <= 0:
        return lp
    n = logits.shape[-1]
    return torch.logaddexp(lp + math.log1p(-unimix), torch.full_like(lp, math.log(unimix / n)))


def normal_log_density(x: torch.Tensor, mean: torch.Tensor, std: torch.Tensor) -> torch.Tensor:
    return -0.5 * ((x - mean) / std) ** 2 - torch.log(std) - 0.5 * math.log(2 * math.pi)


def normal_entropy(std: torch.Tensor) -> torch.Tensor:
    return 0.5 * math.log(2 * math.pi * math.e) + torch.log(std)


def tanh_log_jacobian(raw: torch.Tensor) -> torch.Tensor:
    """``log(1 - tanh(raw)^2)`` in its stable form ``2 (log 2 - raw - softplus(-2 raw))``."""
    return 2.0 * (math.log(2.0) - raw - F.softplus(-2.0 * raw))


def onehot_sample(log_probs: torch.Tensor, generator: Optional[torch.Generator] = None, gumbel: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A one-hot draw from the categorical, its gradient the probabilities' (straight through)."""
    if gumbel is None:
        u = torch.rand(log_probs.shape, generator=generator, device=log_probs.device if generator is None or generator.device.type != "cpu" else "cpu")
        gumbel = -torch.log(-torch.log(u.clamp(1e-20, 1 - 1e-7))).to(log_probs.device)
    index = (log_probs + gumbel).argmax(-1)
    hard = F.one_hot(index, log_probs.shape[-1]).to(log_probs.dtype)
    probs = log_probs.exp()
    return hard + probs - probs.detach()


def categorical_kl(log_p: torch.Tensor, log_q: torch.Tensor) -> torch.Tensor:
    """KL(p || q) of categoricals given as log-probabilities, summed over the last axis."""
    return (log_p.exp() * (log_p - log_q)).sum(-1)
