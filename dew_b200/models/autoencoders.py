"""Autoencoders (the ``AutoEncoder`` protocol: ``encode(x) -> latents``, ``decode(z) -> x``) and a ViT encoder.

Reference: src/dew/nn/autoencoders (VAE family behind an ``AutoEncoder`` protocol), src/dew/nn/vision (ViT / CLIP / SigLIP
encoders).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn.attention import SelfAttention
from ..nn.dit import PatchEmbedding, sincos_2d
from ..nn.layers import LayerNorm
from ..nn.mlp import GeluMLP
from ..utils.registry import register


@register("kl_vae")
class KLAutoEncoder(nn.Module):
    """Convolutional VAE with ``downsample`` 2x stages; ``encode`` returns ``scale * mean`` (or a sample when training)."""

    def __init__(self, channels: int = 3, latent_channels: int = 4, features: int = 64, downsample: int = 3, scale: float = 0.18215):
        super().__init__()
        self.scale, self.latent_channels = scale, latent_channels
        enc, c = [nn.Conv2d(channels, features, 3, padding=1)], features
        for _ in range(downsample):
            enc += [nn.SiLU(), nn.Conv2d(c, c * 2, 3, stride=2, padding=1)]
            c *= 2
        enc += [nn.SiLU(), nn.Conv2d(c, 2 * latent_channels, 3, padding=1)]
        self.encoder = nn.Sequential(*enc)
        dec = [nn.Conv2d(latent_channels, c, 3, padding=1)]
        for _ in range(downsample):
            dec += [nn.SiLU(), nn.Upsample(scale_factor=2, mode="nearest"), nn.Conv2d(c, c // 2, 3, padding=1)]
            c //= 2
        dec += [nn.SiLU(), nn.Conv2d(c, channels, 3, padding=1)]
        self.decoder = nn.Sequential(*dec)

    def moments(self, x):
        return self.encoder(x.permute(0, 3, 1, 2)).chunk(2, 1)

    def encode(self, x, sample: bool = False, generator=None):
        mean, logvar = self.moments(x)
        z = mean + torch.exp(0.5 * logvar.clamp(-30, 20)) * torch.randn(mean.shape, generator=generator, device=mean.device) if sample else mean
        return (z * self.scale).permute(0, 2, 3, 1)

    def decode(self, z):
        return self.decoder((z / self.scale).permute(0, 3, 1, 2)).permute(0, 2, 3, 1)

    def loss(self, x, kl_weight: float = 1e-6):
        mean, logvar = self.moments(x)
        z = mean + torch.exp(0.5 * logvar) * torch.randn_like(mean)
        rec = self.decoder(z).permute(0, 2, 3, 1)
        kl = 0.5 * (mean ** 2 + logvar.exp() - 1 - logvar).mean()
        return F.mse_loss(rec, x) + kl_weight * kl


@register("vit")
class ViT(nn.Module):
    """Vision transformer encoder: NHWC image -> ``[B, tokens, features]`` (pre-norm blocks, sin-cos positions)."""

    def __init__(self, patch_size: int = 16, features: int = 384, num_layers: int = 12, num_heads: int = 6, mlp_ratio: float = 4.0, channels: int = 3):
        super().__init__()
        self.features = features
        self.embed = PatchEmbedding(patch_size, channels, features)
        self.blocks = nn.ModuleList([nn.ModuleDict({"n1": LayerNorm(features), "attn": SelfAttention(features, num_heads, bias=True, causal=False),
                                                    "n2": LayerNorm(features), "mlp": GeluMLP(features, int(features * mlp_ratio), approximate="none")})
                                     for _ in range(num_layers)])
        self.norm = LayerNorm(features)
        self.patch_size = patch_size

    def forward(self, x):
        if x.dim() == 3:                    # already tokens [B, T, d_in]: used as a JEPA context encoder on patch tokens
            t = x
        else:
            B, H, W, _ = x.shape
            t = self.embed(x)
            t = t + sincos_2d(H // self.patch_size, W // self.patch_size, self.features, t.device).to(t.dtype)[None]
        for b in self.blocks:
            t = t + b["attn"](b["n1"](t))
            t = t + b["mlp"](b["n2"](t))
        return self.norm(t)
