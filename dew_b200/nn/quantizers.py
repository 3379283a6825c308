"""Vector quantisers for discrete tokenisers.

``ResidualVQ``  residual vector quantisation (EnCodec / Moshi style): each stage takes the codeword nearest what the stages before
                left (the first on a tie) and subtracts it; decoding sums the chosen codewords; computed in fp32.  Trainable with the
                straight-through estimator and commitment / codebook losses, or with frozen tables
``FSQ``         finite scalar quantisation (arXiv 2309.15505): each of a few channels is bounded by tanh and rounded to ``levels[i]``
                values; the implied codebook is the product grid, no codebook to learn and none to collapse
``LFQ``         lookup-free quantisation: each channel's sign, with the entropy terms that keep the codes used

Reference: src/dew/nn/quantizers.py (residual vector quantisation over frozen tables).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class ResidualVQ(nn.Module):
    def __init__(self, width: int, sizes: Sequence[int] = (1024, 1024, 1024, 1024), beta: float = 0.25):
        super().__init__()
        self.codebooks = nn.ParameterList([nn.Parameter(torch.randn(n, width) / width ** 0.5) for n in sizes])
        self.beta = beta

    @torch.no_grad()
    def encode(self, x: torch.Tensor) -> torch.Tensor:
        """``x [..., width]`` -> codes ``[..., stages]``."""
        r = x.float()
        codes = []
        for table in self.codebooks:
            t = table.float()
            d = (r * r).sum(-1, keepdim=True) - 2 * r @ t.t() + (t * t).sum(-1)
            idx = d.argmin(-1)                                          # argmin returns the first index on a tie
            codes.append(idx)
            r = r - t[idx]
        return torch.stack(codes, -1)

    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        return sum(table.float()[codes[..., s]] for s, table in enumerate(self.codebooks))

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """-> (quantised with a straight-through gradient, codes, loss = codebook + beta * commitment, summed over stages)."""
        r = x.float()
        total = torch.zeros_like(r)
        loss = r.new_zeros(())
        codes = []
        for table in self.codebooks:
            t = table.float()
            d = (r.detach() ** 2).sum(-1, keepdim=True) - 2 * r.detach() @ t.t() + (t * t).sum(-1)
            idx = d.argmin(-1)
            q = t[idx]
            loss = loss + F.mse_loss(q, r.detach()) + self.beta * F.mse_loss(r, q.detach())
            total = total + q
            r = r - q.detach()
            codes.append(idx)
        return (x.float() + (total - x.float()).detach()).to(x.dtype), torch.stack(codes, -1), loss


class FSQ(nn.Module):
    def __init__(self, levels: Sequence[int] = (8, 5, 5, 5)):
        super().__init__()
        self.register_buffer("levels", torch.tensor(list(levels), dtype=torch.float32))
        basis = torch.cumprod(torch.tensor([1] + list(levels[:-1])), 0)
        self.register_buffer("basis", basis)
        self.codebook_size = int(torch.tensor(list(levels)).prod())

    def bound(self, z: torch.Tensor) -> torch.Tensor:
        half = (self.levels - 1) * (1 - 1e-3) / 2
        offset = torch.where(self.levels % 2 == 0, torch.full_like(self.levels, 0.5), torch.zeros_like(self.levels))
        shift = torch.atanh(offset / half)
        return torch.tanh(z.float() + shift) * half - offset

    def forward(self, z: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``z [..., len(levels)]`` -> (quantised in [-1, 1] with a straight-through gradient, code indices)."""
        b = self.bound(z)
        rounded = b + (b.round() - b).detach()
        half_width = torch.div(self.levels, 2, rounding_mode="floor")
        return (rounded / half_width).to(z.dtype), self.codes(rounded)

    def codes(self, rounded: torch.Tensor) -> torch.Tensor:
        half_width = torch.div(self.levels, 2, rounding_mode="floor")
        digits = (rounded.detach() + half_width).round().long()
        return (digits * self.basis).sum(-1)

    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        digits = torch.div(codes[..., None], self.basis, rounding_mode="floor") % self.levels.long()
        half_width = torch.div(self.levels, 2, rounding_mode="floor")
        return (digits.float() - half_width) / half_width


class LFQ(nn.Module):
    def __init__(self, bits: int = 10, entropy_weight: float = 0.1, diversity: float = 1.0, temperature: float = 0.01):
        super().__init__()
        self.bits, self.entropy_weight, self.diversity, self.temperature = bits, entropy_weight, diversity, temperature
        self.register_buffer("basis", 2 ** torch.arange(bits))

    def forward(self, z: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``z [..., bits]`` -> (signs with a straight-through gradient, code indices, entropy loss): the loss lowers each sample's
        code entropy (confident bits) and raises the batch's (all codes used), computed per bit (the codes factorise)."""
        zf = z.float()
        q = torch.where(zf > 0, torch.ones_like(zf), -torch.ones_like(zf))
        codes = ((q > 0).long() * self.basis).sum(-1)
        p = torch.sigmoid(2 * zf / self.temperature)                     # P(bit = 1) under the distance-softmax to +-1
        eps = 1e-8
        per_sample = -(p * (p + eps).log() + (1 - p) * (1 - p + eps).log()).sum(-1).mean()
        mean_p = p.reshape(-1, self.bits).mean(0)
        batch = -(mean_p * (mean_p + eps).log() + (1 - mean_p) * (1 - mean_p + eps).log()).sum()
        loss = self.entropy_weight * (per_sample - self.diversity * batch)
        return (zf + (q - zf).detach()).to(z.dtype), codes, loss
