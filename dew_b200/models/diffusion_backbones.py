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


# ------------------------------------------------------------------------------------------------ more families
@register("unet_3d")
class UNet3D(nn.Module):
    """Video UNet ``[B, T, H, W, C]``: the 2-D UNet's residual blocks run per frame, and after every level a temporal
    attention mixes each location over the frames (factorised space / time, as video diffusion UNets do)."""

    def __init__(self, input_channels=3, output_channels=3, features: Sequence[int] = (32, 64), blocks_per_level: int = 1,
                 text_features: Optional[int] = None, num_classes: Optional[int] = None, heads: int = 4):
        super().__init__()
        temb = features[0] * 4
        self.cond = ConditioningEmbed(temb, text_features, num_classes)
        self.inp = nn.Conv2d(input_channels, features[0], 3, padding=1)
        self.down, self.down_t, self.up, self.up_t = nn.ModuleList(), nn.ModuleList(), nn.ModuleList(), nn.ModuleList()
        self.pool, self.unpool = nn.ModuleList(), nn.ModuleList()
        c = features[0]
        for lvl, f in enumerate(features):
            self.down.append(nn.ModuleList([_ResBlock(c if i == 0 else f, f, temb) for i in range(blocks_per_level)]))
            self.down_t.append(_TemporalAttention(f, heads))
            self.pool.append(nn.Conv2d(f, f, 3, stride=2, padding=1) if lvl < len(features) - 1 else nn.Identity())
            c = f
        self.mid = _ResBlock(c, c, temb)
        for lvl, f in reversed(list(enumerate(features))):
            self.up.append(nn.ModuleList([_ResBlock((c + f) if i == 0 else f, f, temb) for i in range(blocks_per_level)]))
            self.up_t.append(_TemporalAttention(f, heads))
            self.unpool.append(nn.Upsample(scale_factor=2, mode="nearest") if lvl > 0 else nn.Identity())
            c = f
        self.out = nn.Sequential(nn.GroupNorm(min(8, c), c), nn.SiLU(), nn.Conv2d(c, output_channels, 3, padding=1))
        nn.init.zeros_(self.out[-1].weight); nn.init.zeros_(self.out[-1].bias)

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        B, T, H, W, C = x.shape
        t = self.cond(temb, ctx.get("text"), ctx.get("label")).repeat_interleave(T, 0)
        h = self.inp(x.reshape(B * T, H, W, C).permute(0, 3, 1, 2))
        skips = []
        for blocks, mix, pool in zip(self.down, self.down_t, self.pool):
            for b in blocks:
                h = b(h, t)
            h = mix(h, T)
            skips.append(h)
            h = pool(h)
        h = self.mid(h, t)
        for blocks, mix, unpool in zip(self.up, self.up_t, self.unpool):
            s = skips.pop()
            if h.shape[-2:] != s.shape[-2:]:
                h = F.interpolate(h, size=s.shape[-2:], mode="nearest")
            h = torch.cat([h, s], 1)
            for b in blocks:
                h = b(h, t)
            h = unpool(mix(h, T))
        if h.shape[-2:] != (H, W):
            h = F.interpolate(h, size=(H, W), mode="nearest")
        return self.out(h).permute(0, 2, 3, 1).reshape(B, T, H, W, -1).float()


class _TemporalAttention(nn.Module):
    """Self-attention over the frame axis at every pixel of ``[B*T, C, h, w]`` feature maps (residual, zero-initialised out)."""

    def __init__(self, channels: int, heads: int):
        super().__init__()
        self.norm = nn.GroupNorm(min(8, channels), channels)
        self.attn = SelfAttention(channels, heads, bias=True, causal=False)
        self.gate = nn.Parameter(torch.zeros(()))

    def forward(self, x, frames: int):
        BT, C, h, w = x.shape
        B = BT // frames
        seq = self.norm(x).reshape(B, frames, C, h * w).permute(0, 3, 1, 2).reshape(B * h * w, frames, C)
        y = self.attn(seq).reshape(B, h * w, frames, C).permute(0, 2, 3, 1).reshape(BT, C, h, w)
        return x + self.gate * y


@register("hierarchical_mmdit")
class HierarchicalMMDiT(_TokenBackbone):
    """Joint text-image blocks at two resolutions: fine tokens, then 2 x 2 merged coarse tokens (4x fewer, the bulk of the
    depth), then fine again with a skip from the first stage."""

    def __init__(self, patch_size=2, emb_features=128, num_layers=(1, 2, 1), num_heads=4, mlp_ratio=4.0, input_channels=3, output_channels=3,
                 text_features=64, num_classes=None):
        super().__init__(patch_size, emb_features, input_channels, output_channels, text_features, num_classes)
        d = emb_features
        self.text_in = Linear(text_features, d, bias=True)
        mk = lambda n: nn.ModuleList([_JointBlock(d, num_heads, mlp_ratio) for _ in range(n)])
        self.fine_in, self.coarse, self.fine_out = mk(num_layers[0]), mk(num_layers[1]), mk(num_layers[2])
        self.merge = Linear(4 * d, d, bias=True)
        self.split = Linear(d, 4 * d, bias=True)
        self.skip = Linear(2 * d, d, bias=True)

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        img, (gh, gw) = self.tokens(x)
        if gh % 2 or gw % 2:
            raise ValueError("the token grid must be even in both directions to merge 2 x 2 tokens")
        text = ctx.get("text")
        if text is None:
            text = torch.zeros(x.shape[0], 1, self.text_in.in_features, device=x.device)
        c = self.conditioning(temb, text, ctx.get("label"))
        txt = self.text_in(text.to(img.dtype))
        for b in self.fine_in:
            img, txt = b(img, txt, c)
        B, N, d = img.shape
        first = img
        coarse = self.merge(img.reshape(B, gh // 2, 2, gw // 2, 2, d).permute(0, 1, 3, 2, 4, 5).reshape(B, N // 4, 4 * d))
        for b in self.coarse:
            coarse, txt = b(coarse, txt, c)
        fine = self.split(coarse).reshape(B, gh // 2, gw // 2, 2, 2, d).permute(0, 1, 3, 2, 4, 5).reshape(B, N, d)
        img = self.skip(torch.cat([fine, first], -1))
        for b in self.fine_out:
            img, txt = b(img, txt, c)
        return self.output(img, c, (gh, gw))


@register("ssm_dit")
class SSMDiT(HybridDiT):
    """A DiT whose every block is a bidirectional Mamba-2 mixer under adaLN modulation (no attention)."""

    def __init__(self, **kw):
        kw.setdefault("pattern", "mamba2")
        super().__init__(**kw)


@register("jepa_encoder")
class JepaEncoder(nn.Module):
    """ViT encoder over image patches for JEPA: ``images [B, H, W, C]`` or patch tokens -> ``[B, tokens, features]``; ``keep``
    (a bool mask over tokens) runs the blocks on the kept tokens only, the way a context encoder sees a masked image."""

    def __init__(self, patch_size=4, emb_features=128, num_layers=4, num_heads=4, mlp_ratio=4.0, input_channels=3, frames: int = 1):
        super().__init__()
        self.patch_size, self.emb_features, self.frames = patch_size, emb_features, frames
        self.embed = PatchEmbedding(patch_size, input_channels, emb_features)
        self.blocks = nn.ModuleList([nn.ModuleDict({"n1": LayerNorm(emb_features), "attn": SelfAttention(emb_features, num_heads, bias=True, causal=False),
                                                    "n2": LayerNorm(emb_features), "mlp": GeluMLP(emb_features, int(emb_features * mlp_ratio))})
                                     for _ in range(num_layers)])
        self.norm = LayerNorm(emb_features)

    def tokens(self, x):
        if x.dim() == 5:                                   # video: frames are embedded one by one, time added as a second signal
            B, T, H, W, C = x.shape
            tok = self.embed(x.reshape(B * T, H, W, C))
            gh, gw = H // self.patch_size, W // self.patch_size
            tok = tok + sincos_2d(gh, gw, self.emb_features, tok.device).to(tok.dtype)[None]
            tok = tok.reshape(B, T, gh * gw, -1) + sinusoidal(torch.arange(T, device=x.device).float(), self.emb_features).to(tok.dtype)[None, :, None]
            return tok.reshape(B, T * gh * gw, -1)
        B, H, W, C = x.shape
        tok = self.embed(x)
        return tok + sincos_2d(H // self.patch_size, W // self.patch_size, self.emb_features, tok.device).to(tok.dtype)[None]

    def forward(self, x, keep: Optional[torch.Tensor] = None):
        tok = self.tokens(x) if x.dim() >= 4 else x
        if keep is not None:
            tok = tok[:, keep]
        for b in self.blocks:
            tok = tok + b["attn"](b["n1"](tok))
            tok = tok + b["mlp"](b["n2"](tok))
        return self.norm(tok)


@register("jepa_video_encoder")
class JepaVideoEncoder(JepaEncoder):
    """The same encoder over ``[B, T, H, W, C]`` clips (space-time tokens, joint attention)."""

    def __init__(self, frames: int = 8, **kw):
        super().__init__(frames=frames, **kw)
