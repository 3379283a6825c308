"""Kimi delta attention mixer: the gated delta rule with per-channel decay, short convolutions on q / k / v, a low-rank
decay projection, and a gated RMSNorm on the output.  Reference: src/dew/nn/kda.py (319 lines), kernels src/dew/nn/kernels/fla_kda.py."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import scan
from .layers import Linear, declare
from .linear_attention import ShortConv


class KimiDeltaAttention(nn.Module):
    def __init__(self, features: int, num_heads: int = 8, head_dim: int = 64, conv_size: int = 4, decay_rank: int = 32,
                 norm_eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.h, self.d = num_heads, head_dim
        inner = num_heads * head_dim
        kw = dict(dtype=dtype, device=device)
        self.q_proj, self.k_proj, self.v_proj = (Linear(features, inner, axes=("embed", "heads"), **kw) for _ in range(3))
        self.q_conv, self.k_conv, self.v_conv = (ShortConv(inner, conv_size, activation=True, **kw) for _ in range(3))
        self.decay_down = Linear(features, decay_rank, axes=("embed", None), **kw)
        self.decay_up = Linear(decay_rank, inner, axes=(None, "heads"), **kw)
        self.A_log = declare(nn.Parameter(torch.zeros(num_heads, dtype=torch.float32, device=device)), ("heads",), "A_log")
        self.dt_bias = declare(nn.Parameter(torch.zeros(inner, dtype=torch.float32, device=device)), ("heads",), "dt_bias")
        self.beta_proj = Linear(features, num_heads, axes=("embed", "heads"), **kw)
        self.gate_proj = Linear(features, inner, axes=("embed", "heads"), **kw)
        self.norm_weight = declare(nn.Parameter(torch.ones(head_dim, dtype=dtype, device=device)), ("norm",), "scale")
        self.o_proj = Linear(inner, features, axes=("heads", "embed"), **kw)
        self.eps = norm_eps

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0, chunked: bool = True):
        B, T, _ = x.shape
        H, D = self.h, self.d
        q = self.q_conv(self.q_proj(x), segment_ids).view(B, T, H, D)
        k = self.k_conv(self.k_proj(x), segment_ids).view(B, T, H, D)
        v = self.v_conv(self.v_proj(x), segment_ids).view(B, T, H, D)
        q, k = F.normalize(q.float(), dim=-1).to(x.dtype), F.normalize(k.float(), dim=-1).to(x.dtype)
        a = self.decay_up(self.decay_down(x)).float() + self.dt_bias
        g = (-torch.exp(self.A_log.float()).repeat_interleave(D) * F.softplus(a)).view(B, T, H, D)     # <= 0 per channel
        beta = torch.sigmoid(self.beta_proj(x).float())
        fn = scan.kda_chunked if (chunked and T > 1) else scan.kda_recurrent
        o, _ = fn(q, k, v, g, beta)
        z = self.gate_proj(x).view(B, T, H, D)
        o = ops.gated_rms_norm(o.reshape(-1, D), z.reshape(-1, D), self.norm_weight, self.eps).view(B, T, H * D)
        return self.o_proj(o)
