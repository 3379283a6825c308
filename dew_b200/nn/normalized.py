"""The normalised transformer's arithmetic (nGPT, arXiv 2410.01131): hidden states live on the unit sphere and each sublayer's
output joins the residual by a learned step along the sphere.

``justnorm(x)``          x / |x| along the feature axis, reduced in fp32, returned in x's dtype
``sphere_step(h, y, a)`` ``justnorm(h + a * (justnorm(y) - h))``: the residual moves toward the sublayer's normalised output by the
                         per-feature step ``a`` (an "eigen learning rate"), then returns to the sphere
``Scale``                a learned vector stored at ``init / scale`` magnitude and read as ``p * scale / init``: the paper's way of giving
                         a scalar its own effective learning rate
``NormalizedAttention`` / ``NormalizedMLP`` / ``NormalizedBlock``   q and k normalised per head and scaled by ``s_qk`` (softmax scale
                         ``sqrt(d_head)`` instead of its inverse), the MLP's hidden scaled by ``s_u`` / ``s_v * sqrt(d)``
``normalize_weights_``   after every optimizer step each matrix's rows (along the embedding axis) return to unit norm

Reference: src/dew/nn/ngpt.py (``justnorm``, ``slerp_norm``, scaled parameters, the normalised block).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .attention_variants import _causal_mask, biased_attention


def justnorm(x: torch.Tensor, dim: int = -1, eps: float = 0.0) -> torch.Tensor:
    n = x.float().norm(dim=dim, keepdim=True).clamp_min(max(eps, 1e-12))
    return (x.float() / n).to(x.dtype)


def sphere_step(h: torch.Tensor, y: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    h, y = justnorm(h), justnorm(y)
    return justnorm((h.float() + alpha.float().abs() * (y.float() - h.float())).to(h.dtype))


class Scale(nn.Module):
    def __init__(self, width: int, init: float = 1.0, scale: float = 1.0):
        super().__init__()
        self.init, self.scale = init, scale
        self.value = nn.Parameter(torch.full((width,), scale))

    def forward(self) -> torch.Tensor:
        return self.value * (self.init / self.scale)


class NormalizedAttention(nn.Module):
    def __init__(self, features: int, num_heads: int, causal: bool = True):
        super().__init__()
        self.num_heads, self.head_dim, self.causal = num_heads, features // num_heads, causal
        self.qkv = nn.Linear(features, 3 * features, bias=False)
        self.out = nn.Linear(features, features, bias=False)
        self.s_qk = Scale(features, 1.0, features ** -0.5)

    def forward(self, h, cos=None, sin=None, positions=None):
        B, S, d = h.shape
        H, D = self.num_heads, self.head_dim
        q, k, v = self.qkv(h).view(B, S, 3, H, D).unbind(2)
        if cos is not None:
            from .. import ops
            q, k = ops.rope(q, cos, sin, positions), ops.rope(k, cos, sin, positions)
        s = self.s_qk().view(H, D).to(q.dtype)
        q, k = justnorm(q) * s, justnorm(k) * s
        mask = _causal_mask(S, S, h.device)[None, None] if self.causal else None
        out = biased_attention(q, k, v, mask=mask, scale=math.sqrt(D))       # unit vectors: the logits need the larger scale
        return self.out(out.reshape(B, S, d))


class NormalizedMLP(nn.Module):
    def __init__(self, features: int, hidden: int):
        super().__init__()
        self.features = features
        self.up = nn.Linear(features, 2 * hidden, bias=False)
        self.down = nn.Linear(hidden, features, bias=False)
        self.s_u, self.s_v = Scale(hidden, 1.0, 1.0), Scale(hidden, 1.0, 1.0)

    def forward(self, h):
        u, v = self.up(h).chunk(2, -1)
        u = u * self.s_u().to(u.dtype)
        v = v * self.s_v().to(v.dtype) * math.sqrt(self.features)
        return self.down(u * F.silu(v))


class NormalizedBlock(nn.Module):
    def __init__(self, features: int, num_heads: int, hidden: Optional[int] = None, layers: int = 1):
        super().__init__()
        self.attn = NormalizedAttention(features, num_heads)
        self.mlp = NormalizedMLP(features, hidden or 4 * features)
        base = 1.0 / max(1, layers)                                     # the paper's alpha_init ~ 1 / n_layers, stored at 1 / sqrt(d)
        self.alpha_a, self.alpha_m = Scale(features, base, features ** -0.5), Scale(features, base, features ** -0.5)

    def forward(self, h, cos=None, sin=None, positions=None):
        h = sphere_step(h, self.attn(h, cos, sin, positions), self.alpha_a())
        return sphere_step(h, self.mlp(h), self.alpha_m())


@torch.no_grad()
def normalize_weights_(module: nn.Module) -> int:
    """Return every matrix of the normalised sublayers to unit norm along its embedding axis (the axis of size ``features``): the
    input axis of ``qkv`` / ``up``, the output axis of ``out`` / ``down``, rows of an embedding.  Returns how many were normalised."""
    count = 0
    for m in module.modules():
        if isinstance(m, NormalizedAttention):
            pairs = [(m.qkv.weight, 1), (m.out.weight, 0)]
        elif isinstance(m, NormalizedMLP):
            pairs = [(m.up.weight, 1), (m.down.weight, 0)]
        elif isinstance(m, nn.Embedding):
            pairs = [(m.weight, 1)]
        else:
            continue
        for w, dim in pairs:
            w.copy_(justnorm(w, dim=dim))
            count += 1
    return count
