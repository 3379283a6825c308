"""More diffusion backbones behind the same call ``model(x, temb, textcontext=None, train=False)`` (NHWC in / out):
``UNet`` (residual conv blocks, attention at coarse levels), ``UViT`` (ViT with long skip connections), ``SimpleMMDiT``
(joint text-image attention blocks), ``VideoDiT`` (factorised space / time attention), ``SimpleUDiT`` (DiT with U-shaped
skips), ``HybridDiT`` (attention and Mamba-2 blocks interleaved).

Reference families: src/dew/nn/backbones/{unet,uvit,mmdit,video_dit,simple_udit,hybrid_dit}.py (docs/benchmarks.md:26-39).
"""
from __future__ import annotations

import math
from typing import Any, Mapping, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn.attention import SelfAttention
from ..nn.dit import ConditioningEmbed, ModulatedBlock, PatchEmbedding, PatchSequenceOutput, modulate, sincos_2d
from ..nn.layers import LayerNorm, Linear, sinusoidal
from ..nn.mlp import GeluMLP
from ..utils.registry import register


def _ctx(textcontext):
    return textcontext if isinstance(textcontext, Mapping) else {"text": textcontext}


# ------------------------------------------------------------------------------------------------ UNet
class _ResBlock(nn.Module):
    def __init__(self, cin, cout, temb):
        super().__init__()
        self.n1, self.c1 = nn.GroupNorm(min(8, cin), cin), nn.Conv2d(cin, cout, 3, padding=1)
        self.t = nn.Linear(temb, cout)
        self.n2, self.c2 = nn.GroupNorm(min(8, cout), cout), nn.Conv2d(cout, cout, 3, padding=1)
        self.skip = nn.Conv2d(cin, cout, 1) if cin != cout else nn.Identity()

    def forward(self, x, t):
        h = self.c1(F.silu(self.n1(x))) + self.t(t)[:, :, None, None]
        return self.skip(x) + self.c2(F.silu(self.n2(h)))


class _SpatialAttention(nn.Module):
    def __init__(self, c, heads=4):
        super().__init__()
        self.norm, self.attn = nn.GroupNorm(min(8, c), c), SelfAttention(c, heads, bias=True, causal=False)

    def forward(self, x):
        B, C, H, W = x.shape
        t = self.norm(x).reshape(B, C, H * W).transpose(1, 2)
        return x + self.attn(t).transpose(1, 2).reshape(B, C, H, W)


@register("unet")
class UNet(nn.Module):
    def __init__(self, input_channels=3, output_channels=3, features: Sequence[int] = (64, 128, 256), attention_levels: Sequence[int] = (2,),
                 blocks_per_level: int = 2, text_features: Optional[int] = None, num_classes: Optional[int] = None, heads: int = 4):
        super().__init__()
        temb = features[0] * 4
        self.cond = ConditioningEmbed(temb, text_features, num_classes)
        self.inp = nn.Conv2d(input_channels, features[0], 3, padding=1)
        self.down, self.up = nn.ModuleList(), nn.ModuleList()
        chans, c = [features[0]], features[0]
        for lvl, f in enumerate(features):
            for _ in range(blocks_per_level):
                self.down.append(nn.ModuleList([_ResBlock(c, f, temb), _SpatialAttention(f, heads) if lvl in attention_levels else nn.Identity()]))
                c = f
                chans.append(c)
            if lvl < len(features) - 1:
                self.down.append(nn.ModuleList([nn.Conv2d(c, c, 3, stride=2, padding=1), nn.Identity()]))
                chans.append(c)
        self.mid = nn.ModuleList([_ResBlock(c, c, temb), _SpatialAttention(c, heads), _ResBlock(c, c, temb)])
        for lvl, f in reversed(list(enumerate(features))):
            for i in range(blocks_per_level + 1):
                self.up.append(nn.ModuleList([_ResBlock(c + chans.pop(), f, temb), _SpatialAttention(f, heads) if lvl in attention_levels else nn.Identity(),
                                              nn.Upsample(scale_factor=2, mode="nearest") if (i == blocks_per_level and lvl > 0) else nn.Identity()]))
                c = f
        self.out = nn.Sequential(nn.GroupNorm(min(8, c), c), nn.SiLU(), nn.Conv2d(c, output_channels, 3, padding=1))
        nn.init.zeros_(self.out[-1].weight); nn.init.zeros_(self.out[-1].bias)

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        t = self.cond(temb, ctx.get("text"), ctx.get("label"))
        h = self.inp(x.permute(0, 3, 1, 2))
        skips = [h]
        for block, attn in self.down:
            h = block(h, t) if isinstance(block, _ResBlock) else block(h)
            h = attn(h)
            skips.append(h)
        h = self.mid[2](self.mid[1](self.mid[0](h, t)), t)
        for block, attn, up in self.up:
            h = up(attn(block(torch.cat([h, skips.pop()], 1), t)))
        return self.out(h).permute(0, 2, 3, 1).float()


# ------------------------------------------------------------------------------------------------ token backbones
class _TokenBackbone(nn.Module):
    def __init__(self, patch_size, emb_features, input_channels, output_channels, text_features, num_classes):
        super().__init__()
        self.patch_size, self.emb_features = patch_size, emb_features
        self.embed = PatchEmbedding(patch_size, input_channels, emb_features)
        self.conditioning = ConditioningEmbed(emb_features, text_features, num_classes)
        self.output = PatchSequenceOutput(emb_features, patch_size, output_channels)

    def tokens(self, x):
        B, H, W, _ = x.shape
        gh, gw = H // self.patch_size, W // self.patch_size
        t = self.embed(x)
        return t + sincos_2d(gh, gw, self.emb_features, t.device).to(t.dtype)[None], (gh, gw)


@register("uvit")
class UViT(_TokenBackbone):
    """Time is a token; the second half of the blocks concatenates the matching first-half activation (long skips)."""

    def __init__(self, patch_size=4, emb_features=256, num_layers=8, num_heads=4, mlp_ratio=4.0, input_channels=3, output_channels=3,
                 text_features=None, num_classes=None):
        super().__init__(patch_size, emb_features, input_channels, output_channels, text_features, num_classes)
        half = num_layers // 2
        mk = lambda: nn.ModuleDict({"n1": LayerNorm(emb_features), "attn": SelfAttention(emb_features, num_heads, bias=True, causal=False),
                                    "n2": LayerNorm(emb_features), "mlp": GeluMLP(emb_features, int(emb_features * mlp_ratio))})
        self.inb = nn.ModuleList([mk() for _ in range(half)])
        self.midb = mk()
        self.outb = nn.ModuleList([mk() for _ in range(half)])
        self.skips = nn.ModuleList([Linear(2 * emb_features, emb_features, bias=True) for _ in range(half)])

    @staticmethod
    def _block(b, x):
        x = x + b["attn"](b["n1"](x))
        return x + b["mlp"](b["n2"](x))

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        t, grid = self.tokens(x)
        c = self.conditioning(temb, ctx.get("text"), ctx.get("label"))
        t = torch.cat([c[:, None], t], 1)
        saved = []
        for b in self.inb:
            t = self._block(b, t)
            saved.append(t)
        t = self._block(self.midb, t)
        for b, s in zip(self.outb, self.skips):
            t = self._block(b, s(torch.cat([t, saved.pop()], -1)))
        return self.output(t[:, 1:], c, grid)


@register("simple_udit")
class SimpleUDiT(_TokenBackbone):
    """adaLN-Zero DiT blocks with U-shaped skip connections between mirrored depths."""

    def __init__(self, patch_size=4, emb_features=256, num_layers=8, num_heads=4, mlp_ratio=4.0, input_channels=3, output_channels=3,
                 text_features=None, num_classes=None):
        super().__init__(patch_size, emb_features, input_channels, output_channels, text_features, num_classes)
        self.blocks = nn.ModuleList([ModulatedBlock(emb_features, num_heads, mlp_ratio) for _ in range(num_layers)])
        self.skips = nn.ModuleList([Linear(2 * emb_features, emb_features, bias=True) for _ in range(num_layers // 2)])

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        t, grid = self.tokens(x)
        c = self.conditioning(temb, ctx.get("text"), ctx.get("label"))
        n = len(self.blocks)
        saved = []
        for i, b in enumerate(self.blocks):
            if i >= n - n // 2:
                t = self.skips[i - (n - n // 2)](torch.cat([t, saved.pop()], -1))
            t = b(t, c)
            if i < n // 2:
                saved.append(t)
        return self.output(t, c, grid)


class _JointBlock(nn.Module):
    """MMDiT block: text and image streams keep their own norms / MLPs / modulation and attend jointly."""

    def __init__(self, d, heads, mlp_ratio):
        super().__init__()
        self.heads = heads
        for s in ("img", "txt"):
            setattr(self, f"{s}_ada", Linear(d, 6 * d, bias=True, zero_init=True))
            setattr(self, f"{s}_qkv", Linear(d, 3 * d, bias=True))
            setattr(self, f"{s}_o", Linear(d, d, bias=True))
            setattr(self, f"{s}_mlp", GeluMLP(d, int(d * mlp_ratio)))
        self.n = LayerNorm(d, affine=False)

    def forward(self, img, txt, c):
        from .. import ops
        mods, qkvs = {}, {}
        for s, x in (("img", img), ("txt", txt)):
            m = getattr(self, f"{s}_ada")(F.silu(c)).chunk(6, -1)
            mods[s] = m
            qkvs[s] = getattr(self, f"{s}_qkv")(modulate(self.n(x), m[0], m[1]))
        B, Ti, d = img.shape
        joint = torch.cat([qkvs["txt"], qkvs["img"]], 1).reshape(B, -1, 3, self.heads, d // self.heads)
        o = ops.attention(joint[:, :, 0], joint[:, :, 1], joint[:, :, 2], causal=False).reshape(B, -1, d)
        Tt = txt.shape[1]
        outs = {}
        for s, x, part in (("txt", txt, o[:, :Tt]), ("img", img, o[:, Tt:])):
            m = mods[s]
            x = x + m[2].unsqueeze(1) * getattr(self, f"{s}_o")(part)
            outs[s] = x + m[5].unsqueeze(1) * getattr(self, f"{s}_mlp")(modulate(self.n(x), m[3], m[4]))
        return outs["img"], outs["txt"]


@register("simple_mmdit")
class SimpleMMDiT(_TokenBackbone):
    def __init__(self, patch_size=4, emb_features=256, num_layers=6, num_heads=4, mlp_ratio=4.0, input_channels=3, output_channels=3,
                 text_features=64, num_classes=None):
        super().__init__(patch_size, emb_features, input_channels, output_channels, text_features, num_classes)
        self.text_in = Linear(text_features, emb_features, bias=True)
        self.blocks = nn.ModuleList([_JointBlock(emb_features, num_heads, mlp_ratio) for _ in range(num_layers)])

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        img, grid = self.tokens(x)
        text = ctx.get("text")
        if text is None:
            text = torch.zeros(x.shape[0], 1, self.text_in.in_features, device=x.device)
        c = self.conditioning(temb, text, ctx.get("label"))
        txt = self.text_in(text.to(img.dtype))
        for b in self.blocks:
            img, txt = b(img, txt, c)
        return self.output(img, c, grid)


@register("video_dit")
class VideoDiT(_TokenBackbone):
    """Video ``[B, T, H, W, C]``: each block attends over space within a frame, then over time at each location."""

    def __init__(self, patch_size=4, emb_features=256, num_layers=4, num_heads=4, mlp_ratio=4.0, input_channels=3, output_channels=3,
                 text_features=None, num_classes=None, max_frames: int = 64):
        super().__init__(patch_size, emb_features, input_channels, output_channels, text_features, num_classes)
        self.space = nn.ModuleList([ModulatedBlock(emb_features, num_heads, mlp_ratio) for _ in range(num_layers)])
        self.time = nn.ModuleList([ModulatedBlock(emb_features, num_heads, mlp_ratio) for _ in range(num_layers)])
        self.max_frames = max_frames

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        B, T, H, W, C = x.shape
        tok, grid = self.tokens(x.reshape(B * T, H, W, C))
        N, d = tok.shape[1], tok.shape[2]
        tok = tok + sinusoidal(torch.arange(T, device=x.device).float(), d).to(tok.dtype).repeat(B, 1)[:, None]
        c = self.conditioning(temb, ctx.get("text"), ctx.get("label"))
        cs, ct = c.repeat_interleave(T, 0), c.repeat_interleave(N, 0)
        for sb, tb in zip(self.space, self.time):
            tok = sb(tok, cs)
            tt = tok.reshape(B, T, N, d).transpose(1, 2).reshape(B * N, T, d)
            tok = tb(tt, ct).reshape(B, N, T, d).transpose(1, 2).reshape(B * T, N, d)
        out = self.output(tok, cs, grid)
        return out.reshape(B, T, H, W, -1)


@register("hybrid_dit")
class HybridDiT(_TokenBackbone):
    """Attention blocks interleaved with bidirectional Mamba-2 blocks (``pattern`` e.g. "mamba2,mamba2,attn")."""

    def __init__(self, patch_size=4, emb_features=256, num_layers=6, num_heads=4, mlp_ratio=4.0, input_channels=3, output_channels=3,
                 text_features=None, num_classes=None, pattern: str = "mamba2,attn", state_dim: int = 32):
        super().__init__(patch_size, emb_features, input_channels, output_channels, text_features, num_classes)
        from ..nn.mamba2 import Mamba2
        kinds = [pattern.split(",")[i % len(pattern.split(","))] for i in range(num_layers)]
        self.kinds = kinds
        self.blocks = nn.ModuleList([ModulatedBlock(emb_features, num_heads, mlp_ratio) if k == "attn" else
                                     nn.ModuleDict({"norm": LayerNorm(emb_features, affine=False), "ada": Linear(emb_features, 3 * emb_features, bias=True, zero_init=True),
                                                    "fwd": Mamba2(emb_features, state_dim=state_dim, head_dim=32), "bwd": Mamba2(emb_features, state_dim=state_dim, head_dim=32)})
                                     for k in kinds])

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        t, grid = self.tokens(x)
        c = self.conditioning(temb, ctx.get("text"), ctx.get("label"))
        for k, b in zip(self.kinds, self.blocks):
            if k == "attn":
                t = b(t, c)
            else:
                sh, sc, g = b["ada"](F.silu(c)).chunk(3, -1)
                h = modulate(b["norm"](t), sh, sc)
                t = t + g.unsqueeze(1) * (b["fwd"](h) + b["bwd"](h.flip(1)).flip(1))
        return self.output(t, c, grid)
