"""Mamba-1 block: input projection to (x, z), short causal conv + SiLU, input-dependent (dt, B, C), selective scan, gate,
output projection.  Reference: src/dew/nn/mixers/mamba.py (450 lines)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import scan
from .layers import Linear, declare
from .linear_attention import ShortConv


class Mamba(nn.Module):
    def __init__(self, features: int, state_dim: int = 16, expand: int = 2, conv_size: int = 4, dt_rank: int | None = None, dtype=None, device=None):
        super().__init__()
        inner = expand * features
        self.inner, self.n = inner, state_dim
        self.dt_rank = dt_rank or math.ceil(features / 16)
        kw = dict(dtype=dtype, device=device)
        self.in_proj = Linear(features, 2 * inner, **kw)
        self.conv = ShortConv(inner, conv_size, bias=True, activation=True, **kw)
        self.x_proj = Linear(inner, self.dt_rank + 2 * state_dim, **kw)
        self.dt_proj = Linear(self.dt_rank, inner, bias=True, **kw)
        self.A_log = declare(nn.Parameter(torch.log(torch.arange(1, state_dim + 1, dtype=torch.float32, device=device)).repeat(inner, 1)), ("mlp", None), "A_log")
        self.D = declare(nn.Parameter(torch.ones(inner, dtype=torch.float32, device=device)), ("mlp",), "scale")
        self.out_proj = Linear(inner, features, **kw)

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0, chunked: bool = True):
        xz = self.in_proj(x)
        xi, z = xz[..., :self.inner], xz[..., self.inner:]
        xi = self.conv(xi, segment_ids)
        p = self.x_proj(xi)
        dt = F.softplus(self.dt_proj(p[..., :self.dt_rank]).float())
        Bm, Cm = p[..., self.dt_rank:self.dt_rank + self.n], p[..., self.dt_rank + self.n:]
        fn = scan.selective_scan if chunked else scan.selective_scan_reference
        y, _ = fn(xi, dt, -torch.exp(self.A_log.float()), Bm, Cm, self.D, z)
        return self.out_proj(y.to(x.dtype))
