"""``SimpleDiT``: a plain stack of adaLN-Zero attention blocks over image patches.

Fields follow the reference's options (src/dew/nn/dit.py:525-533, src/dew/nn/backbones/dit.py:27-52):
``patch_size=16, emb_features=768, num_layers=12, num_heads=12, mlp_ratio=4, output_channels=3, adaln_silu,
routes (TREAD token routing), patch_bottleneck, interval, time_scale``.
Call: ``model(x, temb, textcontext=None, train=False, duration=None)`` with ``x`` NHWC and ``temb`` the model time.
"""
from __future__ import annotations

from typing import Any, Mapping, Optional, Sequence

import torch
import torch.nn as nn

from ..nn.dit import ConditioningEmbed, ModulatedBlock, PatchEmbedding, PatchSequenceOutput, sincos_2d
from ..utils.registry import register


@register("simple_dit")
class SimpleDiT(nn.Module):
    def __init__(self, patch_size: int = 16, emb_features: int = 768, num_layers: int = 12, num_heads: int = 12,
                 mlp_ratio: float = 4.0, input_channels: int = 3, output_channels: int = 3, adaln_silu: bool = True,
                 text_features: Optional[int] = None, num_classes: Optional[int] = None,
                 routes: Sequence[Sequence[float]] = (), patch_bottleneck: Optional[int] = None,
                 interval: bool = False, time_scale: float = 16.0, guidance_embed: bool = False, dtype=None, device=None):
        super().__init__()
        self.patch_size, self.emb_features, self.num_layers, self.num_heads = patch_size, emb_features, num_layers, num_heads
        self.mlp_ratio, self.input_channels, self.output_channels = mlp_ratio, input_channels, output_channels
        self.routes = tuple(tuple(r) for r in routes)
        self.embed = PatchEmbedding(patch_size, input_channels, emb_features, patch_bottleneck, dtype=dtype, device=device)
        self.conditioning = ConditioningEmbed(emb_features, text_features, num_classes, time_scale, interval, guidance_embed, dtype=dtype, device=device)
        self.blocks = nn.ModuleList([ModulatedBlock(emb_features, num_heads, mlp_ratio, adaln_silu, dtype=dtype, device=device)
                                     for _ in range(num_layers)])
        self.output = PatchSequenceOutput(emb_features, patch_size, output_channels, dtype=dtype, device=device)

    def forward(self, x, temb, textcontext: Any = None, train: bool = False, duration=None):
        conditions = textcontext if isinstance(textcontext, Mapping) else {"text": textcontext}
        B, H, W, _ = x.shape
        gh, gw = H // self.patch_size, W // self.patch_size
        dt = self.embed.proj.weight.dtype
        tokens = self.embed(x.to(dt))
        tokens = tokens + sincos_2d(gh, gw, self.emb_features, tokens.device).to(dt)[None]
        c = self.conditioning(temb, conditions.get("text"), conditions.get("label"), duration, conditions.get("guidance"))
        routed = None
        for i, block in enumerate(self.blocks):
            if train and self.routes:
                for ratio, start, end in self.routes:
                    if i == int(start):   # TREAD: a random subset of tokens skips blocks start..end
                        n = tokens.shape[1]
                        keep = n - int(n * ratio)
                        perm = torch.rand(B, n, device=tokens.device).argsort(1)
                        kept_idx = perm[:, :keep].sort(1).values
                        routed = (tokens, kept_idx, int(end))
                        tokens = torch.gather(tokens, 1, kept_idx[..., None].expand(-1, -1, tokens.shape[-1]))
            tokens = block(tokens, c)
            if routed is not None and i == routed[2]:
                full, kept_idx, _ = routed
                tokens = full.scatter(1, kept_idx[..., None].expand(-1, -1, tokens.shape[-1]), tokens)
                routed = None
        return self.output(tokens, c, (gh, gw))

    def model_flops(self, tokens: int, batch: int = 1) -> float:
        d, L = self.emb_features, self.num_layers
        per_tok = L * (2 * d * 3 * d + 2 * d * d + 4 * d * d * self.mlp_ratio + 2 * 6 * d * d / max(tokens, 1))
        attn = L * 4 * tokens * d
        return batch * tokens * (per_tok + attn)
