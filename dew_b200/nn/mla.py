"""Multi-head latent attention (DeepSeek-V2/V3): keys and values are reconstructed from a small shared latent (the KV
cache holds the latent and one shared rotary key per token), queries optionally from their own latent; each head has a
rotary part and a no-position part.  Reference: src/dew/nn/mla.py (1240 lines)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, RMSNorm


class MultiHeadLatentAttention(nn.Module):
    def __init__(self, features: int, num_heads: int, kv_latent: int = 512, q_latent: Optional[int] = None, nope_dim: int = 128,
                 rope_dim: int = 64, v_dim: int = 128, norm_eps: float = 1e-6, causal: bool = True, dtype=None, device=None):
        super().__init__()
        self.h, self.nope, self.rope, self.vd, self.causal = num_heads, nope_dim, rope_dim, v_dim, causal
        kw = dict(dtype=dtype, device=device)
        qd = num_heads * (nope_dim + rope_dim)
        if q_latent:
            self.q_down, self.q_norm, self.q_up = Linear(features, q_latent, **kw), RMSNorm(q_latent, norm_eps, **kw), Linear(q_latent, qd, **kw)
        else:
            self.q_down, self.q_norm, self.q_up = None, None, Linear(features, qd, **kw)
        self.kv_down = Linear(features, kv_latent + rope_dim, **kw)          # latent | shared rotary key
        self.kv_norm = RMSNorm(kv_latent, norm_eps, **kw)
        self.kv_up = Linear(kv_latent, num_heads * (nope_dim + v_dim), **kw)
        self.o_proj = Linear(num_heads * v_dim, features, **kw)
        self.kv_latent = kv_latent

    def latent(self, x):
        """What a KV cache stores per token: ``(normalised latent [B,T,kv_latent], rotary key [B,T,rope_dim])``."""
        c = self.kv_down(x)
        return self.kv_norm(c[..., :self.kv_latent]), c[..., self.kv_latent:]

    def forward(self, x, cos=None, sin=None, positions=None, segment_ids=None, cache=None, layer: int = 0):
        B, T, _ = x.shape
        H = self.h
        q = self.q_up(x) if self.q_down is None else self.q_up(self.q_norm(self.q_down(x)))
        q = q.view(B, T, H, self.nope + self.rope)
        c, k_rope = self.latent(x)
        kv = self.kv_up(c).view(B, T, H, self.nope + self.vd)
        k_nope, v = kv[..., :self.nope], kv[..., self.nope:]
        q_nope, q_rope = q[..., :self.nope], q[..., self.nope:]
        k_rope = k_rope.view(B, T, 1, self.rope)
        if cos is not None:
            q_rope = ops.rope_reference(q_rope, cos[:, :self.rope // 2], sin[:, :self.rope // 2], positions)
            k_rope = ops.rope_reference(k_rope, cos[:, :self.rope // 2], sin[:, :self.rope // 2], positions)
        qf = torch.cat([q_nope, q_rope], -1)
        kf = torch.cat([k_nope, k_rope.expand(B, T, H, self.rope)], -1)
        # pad v to the key width so one attention call serves both (the extra columns are dropped)
        scale = (self.nope + self.rope) ** -0.5
        vpad = torch.nn.functional.pad(v, (0, self.nope + self.rope - self.vd)) if self.vd < self.nope + self.rope else v
        o = ops.attention(qf, kf, vpad, causal=self.causal, scale=scale, segment_ids=segment_ids)[..., :self.vd]
        return self.o_proj(o.reshape(B, T, H * self.vd))
