"""DiT building blocks: patch embedding, 2-D sin-cos positions, conditioning embed, adaLN-Zero block, output head.

Capability parity: src/dew/nn/dit.py (``PatchEmbedding:134``, ``AdaLNParams:183``, ``ConditioningEmbed:246``,
``PatchSequenceOutput:309`` zero-init head, ``ModulatedBlock:572-727``: adaLN-Zero x6, LayerNorm without affine,
QKV bias, tanh-GELU MLP).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .attention import SelfAttention
from .layers import LayerNorm, Linear, sinusoidal
from .mlp import GeluMLP


def sincos_2d(h: int, w: int, dim: int, device=None) -> torch.Tensor:
    """``[h*w, dim]`` fixed 2-D sin-cos position signal (half the channels per axis)."""
    def axis(n, d):
        pos = torch.arange(n, dtype=torch.float32, device=device)
        omega = 1.0 / (10000 ** (torch.arange(d // 2, dtype=torch.float32, device=device) / (d // 2)))
        out = pos[:, None] * omega[None]
        return torch.cat([out.sin(), out.cos()], 1)
    eh, ew = axis(h, dim // 2), axis(w, dim // 2)
    grid = torch.cat([eh[:, None, :].expand(h, w, -1), ew[None, :, :].expand(h, w, -1)], -1)
    return grid.reshape(h * w, dim)


class PatchEmbedding(nn.Module):
    """NHWC image -> ``[B, tokens, features]`` with a strided patch projection (a GEMM over flattened patches)."""

    def __init__(self, patch_size: int, in_channels: int, features: int, bottleneck: Optional[int] = None, dtype=None, device=None):
        super().__init__()
        self.patch_size, self.in_channels = patch_size, in_channels
        inner = bottleneck or features
        self.proj = Linear(patch_size * patch_size * in_channels, inner, bias=bottleneck is None, axes=("patch", "embed"), dtype=dtype, device=device)
        self.expand = Linear(inner, features, bias=True, axes=("patch", "embed"), dtype=dtype, device=device) if bottleneck else None

    def forward(self, x):
        B, H, W, C = x.shape
        p = self.patch_size
        assert H % p == 0 and W % p == 0, "image dimensions must be divisible by the patch size"
        x = x.reshape(B, H // p, p, W // p, p, C).permute(0, 1, 3, 2, 4, 5).reshape(B, (H // p) * (W // p), p * p * C)
        x = self.proj(x)
        return self.expand(x) if self.expand is not None else x


class ConditioningEmbed(nn.Module):
    """Time (Fourier -> MLP) plus optional pooled text / class conditioning -> one vector per example."""

    def __init__(self, features: int, text_features: Optional[int] = None, num_classes: Optional[int] = None,
                 time_scale: float = 16.0, interval: bool = False, guidance_embed: bool = False, dtype=None, device=None):
        super().__init__()
        self.features, self.time_scale, self.interval = features, time_scale, interval
        # a guidance-distilled student reads its guidance scale beside the time (as FLUX.1 [dev] does)
        self.g1 = Linear(features, features, bias=True, dtype=dtype, device=device) if guidance_embed else None
        self.g2 = Linear(features, features, bias=True, zero_init=True, dtype=dtype, device=device) if guidance_embed else None
        self.t1 = Linear(features, features, bias=True, dtype=dtype, device=device)
        self.t2 = Linear(features, features, bias=True, dtype=dtype, device=device)
        self.d1 = Linear(features, features, bias=True, dtype=dtype, device=device) if interval else None
        self.text = Linear(text_features, features, bias=True, dtype=dtype, device=device) if text_features else None
        self.classes = nn.Embedding(num_classes + 1, features, dtype=dtype, device=device) if num_classes else None
        self.num_classes = num_classes

    def forward(self, t, context=None, labels=None, duration=None, guidance=None):
        dt = self.t1.weight.dtype
        c = self.t2(F.silu(self.t1(sinusoidal(t, self.features, scale=self.time_scale).to(dt))))
        if self.g1 is not None and guidance is not None:
            c = c + self.g2(F.silu(self.g1(sinusoidal(guidance, self.features, scale=self.time_scale).to(dt))))
        if self.d1 is not None and duration is not None:
            c = c + self.d1(sinusoidal(duration, self.features, scale=self.time_scale).to(dt))
        if self.text is not None and context is not None:
            pooled = context.mean(1) if context.dim() == 3 else context
            c = c + self.text(pooled.to(dt))
        if self.classes is not None and labels is not None:
            c = c + self.classes(labels)
        return c


def modulate(x, shift, scale):
    return x * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


class ModulatedBlock(nn.Module):
    """adaLN-Zero transformer block: six modulation vectors from the conditioning, zero-initialised."""

    def __init__(self, features: int, num_heads: int, mlp_ratio: float = 4.0, adaln_silu: bool = True, dtype=None, device=None):
        super().__init__()
        self.norm1 = LayerNorm(features, affine=False)
        self.attn = SelfAttention(features, num_heads, bias=True, causal=False, dtype=dtype, device=device)
        self.norm2 = LayerNorm(features, affine=False)
        self.mlp = GeluMLP(features, int(features * mlp_ratio), dtype=dtype, device=device)
        self.ada_proj = Linear(features, 6 * features, bias=True, zero_init=True, axes=("embed", "modulation"), dtype=dtype, device=device)
        self.adaln_silu = adaln_silu

    def forward(self, x, c):
        m = self.ada_proj(F.silu(c) if self.adaln_silu else c)
        s1, sc1, g1, s2, sc2, g2 = m.chunk(6, -1)
        x = x + g1.unsqueeze(1) * self.attn(modulate(self.norm1(x), s1, sc1))
        x = x + g2.unsqueeze(1) * self.mlp(modulate(self.norm2(x), s2, sc2))
        return x


class PatchSequenceOutput(nn.Module):
    """Final adaLN + zero-initialised projection back to pixels, then un-patchify to NHWC."""

    def __init__(self, features: int, patch_size: int, out_channels: int, dtype=None, device=None):
        super().__init__()
        self.patch_size, self.out_channels = patch_size, out_channels
        self.norm = LayerNorm(features, affine=False)
        self.ada_proj = Linear(features, 2 * features, bias=True, zero_init=True, dtype=dtype, device=device)
        self.out = Linear(features, patch_size * patch_size * out_channels, bias=True, zero_init=True, dtype=dtype, device=device)

    def forward(self, x, c, grid):
        shift, scale = self.ada_proj(F.silu(c)).chunk(2, -1)
        x = self.out(modulate(self.norm(x), shift, scale)).float()
        B = x.shape[0]
        gh, gw = grid
        p, C = self.patch_size, self.out_channels
        return x.reshape(B, gh, gw, p, p, C).permute(0, 1, 3, 2, 4, 5).reshape(B, gh * p, gw * p, C)
