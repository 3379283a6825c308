"""Fourier feature pyramids: learnable periodic feature grids at coarse-to-fine resolutions, read at any coordinate by
trigonometric (Fourier) interpolation, for coordinate networks (physics-informed networks, neural fields).

Level ``l`` holds a grid of ``features`` channels at resolution ``n_l`` per axis; at a coordinate ``x`` in ``[0, 1)^d`` it is read as its
trigonometric interpolant ``g_l(x) = Re(sum_k theta_hat_l[k] exp(2 pi i k . x))``, ``theta_hat_l`` the grid's DFT over its size - exact
at the grid points, smooth and periodic between them, and differentiable in ``x`` to any order (what a PDE residual needs).  The
levels' reads are concatenated.  ``fourier_features`` is the fixed random-frequency encoding for comparison.

Reference: src/dew/nn/fourier.py (feature pyramids read by Fourier interpolation).
"""
from __future__ import annotations

import math
from typing import Sequence

import torch
import torch.nn as nn


def _frequencies(n: int, device) -> torch.Tensor:
    """Integer frequencies of an ``n``-point DFT in its own order (0, 1, ..., -1); an even size's Nyquist term is kept once."""
    return torch.fft.fftfreq(n, 1.0 / n, device=device)


class FourierFeaturePyramid(nn.Module):
    def __init__(self, dims: int = 2, features: int = 4, resolutions: Sequence[int] = (4, 8, 16), init: float = 1e-2):
        super().__init__()
        if dims not in (1, 2, 3):
            raise ValueError("feature pyramids cover 1 to 3 coordinates")
        self.dims, self.features, self.resolutions = dims, features, tuple(resolutions)
        self.grids = nn.ParameterList([nn.Parameter(torch.randn(features, *([n] * dims)) * init) for n in resolutions])
        self.out_features = features * len(self.resolutions)

    def read(self, level: int, x: torch.Tensor) -> torch.Tensor:
        """``x [N, dims]`` in [0, 1) -> ``[N, features]``."""
        grid = self.grids[level]
        n = self.resolutions[level]
        spec = torch.fft.fftn(grid.to(torch.float32), dim=tuple(range(1, self.dims + 1))) / (n ** self.dims)      # [F, n, ...]
        k = _frequencies(n, x.device)
        # separable phases: exp(2 pi i k_a x_a) per axis, contracted axis by axis
        out = spec.to(torch.complex64)[None].expand(x.shape[0], *spec.shape)                                       # [N, F, n, ...]
        for a in range(self.dims - 1, -1, -1):
            phase = torch.exp(2j * math.pi * k[None, :] * x[:, a:a + 1].to(torch.float32))                          # [N, n]
            if n % 2 == 0:
                # the Nyquist term of an even grid is real at the grid points; read it as a cosine so the interpolant stays real
                phase = phase.clone()
                phase[:, n // 2] = torch.cos(math.pi * n * x[:, a].to(torch.float32)).to(phase.dtype)
            shape = [x.shape[0], 1] + [1] * a + [n]
            out = (out * phase.reshape(shape)).sum(-1)
        return out.real

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        flat = x.reshape(-1, self.dims)
        return torch.cat([self.read(l, flat) for l in range(len(self.resolutions))], -1).reshape(*x.shape[:-1], self.out_features)


def fourier_features(x: torch.Tensor, frequencies: torch.Tensor) -> torch.Tensor:
    """``[sin(2 pi x B), cos(2 pi x B)]`` for a fixed frequency matrix ``B [dims, m]``."""
    proj = 2 * math.pi * x @ frequencies
    return torch.cat([torch.sin(proj), torch.cos(proj)], -1)
