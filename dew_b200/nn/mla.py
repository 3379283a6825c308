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
                 rope_dim: int = 64, v_dim: int = 128, norm_eps: float = 1e-6, causal: bool = True, softmax_gain: float = 1.0,
                 dtype=None, device=None):
        super().__init__()
        # softmax_gain multiplies the (nope + rope) ** -0.5 scale: DeepSeek-V3's long-context releases raise it by YaRN's magnitude squared
        self.softmax_gain = float(softmax_gain)
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

    def _rotate(self, t, cos, sin, positions):
        """Rotary embedding of the ``rope_dim``-wide part: the kernel on a GPU (in place on a fresh contiguous copy), the
        PyTorch form elsewhere."""
        if cos is None:
            return t
        half = self.rope // 2
        tables = self.__dict__.get("_tables")
        if tables is None or tables[0] is not cos:
            tables = (cos, cos[:, :half].contiguous(), sin[:, :half].contiguous())
            self.__dict__["_tables"] = tables
        _, c, s = tables
        if t.is_cuda and t.dtype == torch.bfloat16:
            return ops.rope(t.contiguous(), c, s, positions, rot_heads=t.shape[2])
        return ops.rope_reference(t, c, s, positions)

    def _absorbed(self, q_nope, q_rope, latents, positions, lengths):
        """Attention against cached latents without rebuilding keys or values: the key up-projection is folded into the
        query (``q W_uk``) and the value up-projection is applied after the weighted sum of latents, so a step reads
        ``kv_latent + rope_dim`` numbers per cached token, shared by all heads.
        ``latents [R, L, kv_latent + rope_dim]``; ``positions [R, S]`` absolute; returns ``[R, S, H, v_dim]``."""
        R, S, H, _ = q_nope.shape
        w = self.kv_up.weight.view(H, self.nope + self.vd, self.kv_latent)
        w_uk, w_uv = w[:, :self.nope], w[:, self.nope:]                            # [H, nope, l], [H, vd, l]
        c, k_rope = latents[..., :self.kv_latent].float(), latents[..., self.kv_latent:].float()
        q_lat = torch.einsum("rshn,hnl->rshl", q_nope.float(), w_uk.float())
        scores = torch.einsum("rshl,rtl->rsht", q_lat, c) + torch.einsum("rshd,rtd->rsht", q_rope.float(), k_rope)
        scores = scores * (self.softmax_gain * (self.nope + self.rope) ** -0.5)
        t = torch.arange(latents.shape[1], device=latents.device)
        visible = (t[None, None, :] <= positions[:, :, None]) if self.causal else (t[None, None, :] < lengths[:, None, None])
        visible = visible & (t[None, None, :] < lengths[:, None, None])
        scores = scores.masked_fill(~visible[:, :, None, :], float("-inf"))
        p = torch.nan_to_num(torch.softmax(scores, -1))
        o_lat = torch.einsum("rsht,rtl->rshl", p, c)
        return torch.einsum("rshl,hvl->rshv", o_lat, w_uv.float()).to(q_nope.dtype)

    def forward(self, x, cos=None, sin=None, positions=None, segment_ids=None, cache=None, layer: int = 0):
        B, T, _ = x.shape
        H = self.h
        q = self.q_up(x) if self.q_down is None else self.q_up(self.q_norm(self.q_down(x)))
        q = q.view(B, T, H, self.nope + self.rope)
        c, k_rope = self.latent(x)
        q_nope, q_rope = q[..., :self.nope], q[..., self.nope:]
        k_rope = k_rope.view(B, T, 1, self.rope)
        q_rope = self._rotate(q_rope, cos, sin, positions)
        k_rope = self._rotate(k_rope, cos, sin, positions)
        if cache is not None and hasattr(cache, "write_latent"):
            # the cache holds, per token, the normalised latent and the rotated shared key: kv_latent + rope_dim numbers
            # instead of 2 * heads * head_dim
            if positions is None:
                positions = torch.arange(T, device=x.device)[None].expand(B, T)
            width = self.kv_latent + self.rope
            cache.write_latent(layer, torch.cat([c, k_rope[:, :, 0]], -1), positions)
            lengths = positions.max(1).values + 1
            total = int(lengths.max())
            latents = cache.read_latent(layer, width, total)
            o = self._absorbed(q_nope, q_rope, latents, positions.clamp_min(0), lengths)
            return self.o_proj(o.reshape(B, T, H * self.vd))
        kv = self.kv_up(c).view(B, T, H, self.nope + self.vd)
        k_nope, v = kv[..., :self.nope], kv[..., self.nope:]
        qf = torch.cat([q_nope, q_rope], -1)
        kf = torch.cat([k_nope, k_rope.expand(B, T, H, self.rope)], -1)
        # pad v to the key width so one attention call serves both (the extra columns are dropped)
        scale = self.softmax_gain * (self.nope + self.rope) ** -0.5
        vpad = torch.nn.functional.pad(v, (0, self.nope + self.rope - self.vd)) if self.vd < self.nope + self.rope else v
        o = ops.attention(qf, kf, vpad, causal=self.causal, scale=scale, segment_ids=segment_ids)[..., :self.vd]
        return self.o_proj(o.reshape(B, T, H * self.vd))
