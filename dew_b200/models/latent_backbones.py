"""The released text-to-image / text-to-video transformer families as architectures, behind the backbone call
``model(x, temb, textcontext=None, train=False)`` (NHWC latents in / out; ``textcontext`` a mapping with ``text`` [B, T, d_text],
``pooled`` [B, d_pooled] and, for guidance-distilled models, ``guidance`` [B]):

``RectifiedFlowTransformer``   the FLUX.1 shape: N double-stream blocks (text and image keep their own weights, attend jointly)
                               followed by M single-stream blocks (fused attention + MLP over the concatenated sequence),
                               per-head RMS-normed queries / keys, rotary positions over (frame, row, column) axes, conditioning
                               vector = time (+ guidance) + pooled text.  ``flux``, ``flux2`` (one modulation shared by all blocks,
                               no biases), ``qwen_image`` (double-stream only), ``z_image`` (single-stream only) are registered
                               presets of it.
``SD3Transformer``             MMDiT: joint blocks with learned-free 2-D sin-cos positions on the image tokens, optional q / k norms
                               (SD3.5), the last block's text stream only feeds attention ("pre-only").
``WanTransformer``             video DiT: 3-D patches, self-attention with 3-axis rotary positions, cross-attention to the text
                               states, one time-modulation vector plus a learned per-block offset.
``EDM2UNet``                   the magnitude-preserving U-Net of EDM2: weight-normalised convolutions without biases,
                               magnitude-preserving SiLU / sums / concatenations, pixel-norm attention, learned log-variance head.

They are the architectures, sized by their arguments; released weights load only through loaders that name their tensors
(none is verified here without the releases at hand).

Reference: src/dew/nn/backbones/{flux,flux2,sd3,wan,qwen_image,z_image,edm2}.py (docs/models.md).
"""
from __future__ import annotations

import math
from typing import Mapping, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..nn.dit import modulate, sincos_2d
from ..nn.layers import LayerNorm, Linear, RMSNorm, sinusoidal
from ..utils.registry import register


def _ctx(textcontext) -> Mapping:
    if textcontext is None:
        return {}
    return textcontext if isinstance(textcontext, Mapping) else {"text": textcontext}


# ------------------------------------------------------------------------------------------------ rotary over several axes
def axis_rope(ids: torch.Tensor, dims: Sequence[int], theta: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """``ids [B, T, axes]`` (integer coordinates per axis) -> cos, sin ``[B, T, sum(dims) / 2]``: each axis rotates its own
    slice of the head dimension."""
    cs, sn = [], []
    for a, d in enumerate(dims):
        freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=ids.device) / d))
        ang = ids[..., a].float()[..., None] * freq
        cs.append(ang.cos())
        sn.append(ang.sin())
    return torch.cat(cs, -1), torch.cat(sn, -1)


def apply_axis_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Interleaved-pair rotation (pairs ``(2i, 2i + 1)``) of ``x [B, T, H, D]`` by ``cos, sin [B, T, D / 2]``."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    c, s = cos[:, :, None, :], sin[:, :, None, :]
    out = torch.stack([xf[..., 0] * c - xf[..., 1] * s, xf[..., 0] * s + xf[..., 1] * c], -1)
    return out.reshape(x.shape).to(x.dtype)


def grid_ids(B: int, frames: int, gh: int, gw: int, device) -> torch.Tensor:
    f, h, w = torch.meshgrid(torch.arange(frames, device=device), torch.arange(gh, device=device), torch.arange(gw, device=device), indexing="ij")
    return torch.stack([f, h, w], -1).reshape(1, -1, 3).expand(B, -1, -1)


class _VectorEmbed(nn.Module):
    """Fourier features of a scalar (time, guidance scale) or a pooled vector -> the conditioning width."""

    def __init__(self, d_in: int, d: int, bias: bool = True):
        super().__init__()
        self.fc1, self.fc2 = Linear(d_in, d, bias=bias), Linear(d, d, bias=bias)

    def forward(self, v):
        return self.fc2(F.silu(self.fc1(v)))


class _QKNorm(nn.Module):
    def __init__(self, head_dim: int):
        super().__init__()
        self.q, self.k = RMSNorm(head_dim), RMSNorm(head_dim)

    def forward(self, q, k):
        return self.q(q), self.k(k)


# ------------------------------------------------------------------------------------------------ FLUX-shaped
class _DoubleBlock(nn.Module):
    def __init__(self, d: int, heads: int, mlp_ratio: float, bias: bool, own_modulation: bool, text_pre_only: bool = False):
        super().__init__()
        self.heads, self.text_pre_only = heads, text_pre_only          # the last block of a double-stream-only model: its text output is never read
        for s in ("img", "txt"):
            if own_modulation:
                setattr(self, f"{s}_mod", Linear(d, 6 * d, bias=bias, zero_init=True))
            setattr(self, f"{s}_qkv", Linear(d, 3 * d, bias=bias))
            setattr(self, f"{s}_qknorm", _QKNorm(d // heads))
            if s == "txt" and text_pre_only:
                continue
            setattr(self, f"{s}_proj", Linear(d, d, bias=bias))
            setattr(self, f"{s}_fc1", Linear(d, int(d * mlp_ratio), bias=bias))
            setattr(self, f"{s}_fc2", Linear(int(d * mlp_ratio), d, bias=bias))
        self.norm = LayerNorm(d, affine=False)
        self.own_modulation = own_modulation

    def forward(self, img, txt, vec, cos, sin, shared=None):
        B, Ti, d = img.shape
        Tt = txt.shape[1]
        H = self.heads
        mods, q, k, v = {}, [], [], []
        for s, x in (("txt", txt), ("img", img)):
            m = (getattr(self, f"{s}_mod")(F.silu(vec)) if self.own_modulation else shared[s]).chunk(6, -1)
            mods[s] = m
            qkv = getattr(self, f"{s}_qkv")(modulate(self.norm(x), m[0], m[1])).view(B, -1, 3, H, d // H)
            qs, ks = getattr(self, f"{s}_qknorm")(qkv[:, :, 0], qkv[:, :, 1])
            q.append(qs), k.append(ks), v.append(qkv[:, :, 2])
        q, k, v = torch.cat(q, 1), torch.cat(k, 1), torch.cat(v, 1)
        q, k = apply_axis_rope(q, cos, sin), apply_axis_rope(k, cos, sin)
        o = ops.attention(q, k, v, causal=False).reshape(B, Tt + Ti, d)
        outs = {}
        for s, x, part in (("txt", txt, o[:, :Tt]), ("img", img, o[:, Tt:])):
            if s == "txt" and self.text_pre_only:
                outs[s] = x
                continue
            m = mods[s]
            x = x + m[2].unsqueeze(1) * getattr(self, f"{s}_proj")(part)
            h = getattr(self, f"{s}_fc2")(F.gelu(getattr(self, f"{s}_fc1")(modulate(self.norm(x), m[3], m[4])), approximate="tanh"))
            outs[s] = x + m[5].unsqueeze(1) * h
        return outs["img"], outs["txt"]


class _SingleBlock(nn.Module):
    """Attention and MLP read the same modulated input and share one output projection."""

    def __init__(self, d: int, heads: int, mlp_ratio: float, bias: bool, own_modulation: bool):
        super().__init__()
        self.heads, self.hidden = heads, int(d * mlp_ratio)
        self.mod = Linear(d, 3 * d, bias=bias, zero_init=True) if own_modulation else None
        self.linear1 = Linear(d, 3 * d + self.hidden, bias=bias)
        self.linear2 = Linear(d + self.hidden, d, bias=bias)
        self.qknorm = _QKNorm(d // heads)
        self.norm = LayerNorm(d, affine=False)

    def forward(self, x, vec, cos, sin, shared=None):
        B, T, d = x.shape
        H = self.heads
        shift, scale, gate = (self.mod(F.silu(vec)) if self.mod is not None else shared["single"]).chunk(3, -1)
        qkv, mlp = self.linear1(modulate(self.norm(x), shift, scale)).split([3 * d, self.hidden], -1)
        qkv = qkv.view(B, T, 3, H, d // H)
        q, k = self.qknorm(qkv[:, :, 0], qkv[:, :, 1])
        q, k = apply_axis_rope(q, cos, sin), apply_axis_rope(k, cos, sin)
        o = ops.attention(q, k, qkv[:, :, 2], causal=False).reshape(B, T, d)
        return x + gate.unsqueeze(1) * self.linear2(torch.cat([o, F.gelu(mlp, approximate="tanh")], -1))


@register("flux")
class RectifiedFlowTransformer(nn.Module):
    def __init__(self, patch_size: int = 2, input_channels: int = 16, output_channels: Optional[int] = None, emb_features: int = 256,
                 num_heads: int = 4, double_layers: int = 2, single_layers: int = 4, mlp_ratio: float = 4.0, text_features: int = 64,
                 pooled_features: Optional[int] = 32, guidance_embed: bool = False, axes_dims: Optional[Sequence[int]] = None,
                 theta: float = 10000.0, bias: bool = True, shared_modulation: bool = False):
        super().__init__()
        d, hd = emb_features, emb_features // num_heads
        self.patch, self.cout = patch_size, output_channels or input_channels
        self.axes = tuple(axes_dims) if axes_dims is not None else _default_axes(hd)
        if sum(self.axes) != hd or any(a % 2 for a in self.axes):
            raise ValueError(f"the rotary axes {self.axes} must be even and sum to the head width {hd}")
        self.theta = theta
        self.img_in = Linear(input_channels * patch_size ** 2, d, bias=bias)
        self.txt_in = Linear(text_features, d, bias=bias)
        self.time_in = _VectorEmbed(256, d, bias)
        self.guidance_in = _VectorEmbed(256, d, bias) if guidance_embed else None
        self.vector_in = _VectorEmbed(pooled_features, d, bias) if pooled_features else None
        own = not shared_modulation
        self.double_blocks = nn.ModuleList([_DoubleBlock(d, num_heads, mlp_ratio, bias, own, text_pre_only=(single_layers == 0 and i == double_layers - 1))
                                            for i in range(double_layers)])
        self.single_blocks = nn.ModuleList([_SingleBlock(d, num_heads, mlp_ratio, bias, own) for _ in range(single_layers)])
        if shared_modulation:            # FLUX.2: one set of modulation vectors for every block of a kind
            self.shared_img, self.shared_txt = Linear(d, 6 * d, bias=bias, zero_init=True), Linear(d, 6 * d, bias=bias, zero_init=True)
            self.shared_single = Linear(d, 3 * d, bias=bias, zero_init=True)
        self.shared_modulation = shared_modulation
        self.final_norm = LayerNorm(d, affine=False)
        self.final_mod = Linear(d, 2 * d, bias=bias, zero_init=True)
        self.final = Linear(d, self.cout * patch_size ** 2, bias=bias, zero_init=True)

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        B, Hh, Ww, C = x.shape
        p = self.patch
        gh, gw = Hh // p, Ww // p
        img = self.img_in(x.reshape(B, gh, p, gw, p, C).permute(0, 1, 3, 2, 4, 5).reshape(B, gh * gw, p * p * C).to(self.img_in.weight.dtype))
        text = ctx.get("text")
        if text is None:
            text = torch.zeros(B, 1, self.txt_in.in_features, device=x.device, dtype=img.dtype)
        txt = self.txt_in(text.to(img.dtype))
        vec = self.time_in(sinusoidal(temb * 1000.0, 256).to(img.dtype))
        if self.guidance_in is not None:
            g = ctx.get("guidance")
            g = torch.ones(B, device=x.device) if g is None else g
            vec = vec + self.guidance_in(sinusoidal(g * 1000.0, 256).to(img.dtype))
        if self.vector_in is not None and ctx.get("pooled") is not None:
            vec = vec + self.vector_in(ctx["pooled"].to(img.dtype))
        ids = torch.cat([torch.zeros(B, txt.shape[1], 3, device=x.device, dtype=torch.long), grid_ids(B, 1, gh, gw, x.device)], 1)
        cos, sin = axis_rope(ids, self.axes, self.theta)
        shared = None
        if self.shared_modulation:
            sv = F.silu(vec)
            shared = {"img": self.shared_img(sv), "txt": self.shared_txt(sv), "single": self.shared_single(sv)}
        for blk in self.double_blocks:
            img, txt = blk(img, txt, vec, cos, sin, shared)
        seq = torch.cat([txt, img], 1)
        for blk in self.single_blocks:
            seq = blk(seq, vec, cos, sin, shared)
        img = seq[:, txt.shape[1]:]
        shift, scale = self.final_mod(F.silu(vec)).chunk(2, -1)
        out = self.final(modulate(self.final_norm(img), shift, scale)).float()
        return out.reshape(B, gh, gw, p, p, self.cout).permute(0, 1, 3, 2, 4, 5).reshape(B, Hh, Ww, self.cout)


def _default_axes(hd: int) -> Tuple[int, int, int]:
    """(frame, row, column) slices of the head width in FLUX's proportions (16 : 56 : 56 of 128), even and summing to ``hd``."""
    a = max(2, (hd // 8) // 2 * 2)
    b = ((hd - a) // 2) // 2 * 2
    return (hd - 2 * b, b, b)


@register("flux2")
class Flux2(RectifiedFlowTransformer):
    def __init__(self, **kw):
        super().__init__(**{"bias": False, "shared_modulation": True, "pooled_features": None, "guidance_embed": True, **kw})


@register("qwen_image")
class QwenImage(RectifiedFlowTransformer):
    """Double-stream blocks only; the text states come from a language model and there is no pooled vector."""

    def __init__(self, **kw):
        super().__init__(**{"single_layers": 0, "double_layers": 6, "pooled_features": None, **kw})


@register("z_image")
class ZImage(RectifiedFlowTransformer):
    """Single-stream: text and image tokens share every block."""

    def __init__(self, **kw):
        super().__init__(**{"double_layers": 0, "single_layers": 8, "pooled_features": None, **kw})


# ------------------------------------------------------------------------------------------------ SD3
class _SD3Block(nn.Module):
    def __init__(self, d: int, heads: int, mlp_ratio: float, qk_norm: bool, context_pre_only: bool):
        super().__init__()
        self.heads, self.pre_only = heads, context_pre_only
        self.img_mod = Linear(d, 6 * d, bias=True, zero_init=True)
        self.txt_mod = Linear(d, (2 if context_pre_only else 6) * d, bias=True, zero_init=True)
        self.img_qkv, self.txt_qkv = Linear(d, 3 * d, bias=True), Linear(d, 3 * d, bias=True)
        self.img_qk = _QKNorm(d // heads) if qk_norm else None
        self.txt_qk = _QKNorm(d // heads) if qk_norm else None
        self.img_proj = Linear(d, d, bias=True)
        self.img_fc1, self.img_fc2 = Linear(d, int(d * mlp_ratio), bias=True), Linear(int(d * mlp_ratio), d, bias=True)
        if not context_pre_only:
            self.txt_proj = Linear(d, d, bias=True)
            self.txt_fc1, self.txt_fc2 = Linear(d, int(d * mlp_ratio), bias=True), Linear(int(d * mlp_ratio), d, bias=True)
        self.norm = LayerNorm(d, affine=False)

    def forward(self, img, txt, c):
        B, Ti, d = img.shape
        Tt, H = txt.shape[1], self.heads
        mi = self.img_mod(F.silu(c)).chunk(6, -1)
        mt = self.txt_mod(F.silu(c)).chunk(2 if self.pre_only else 6, -1)
        qi = self.img_qkv(modulate(self.norm(img), mi[0], mi[1])).view(B, Ti, 3, H, d // H)
        qt = self.txt_qkv(modulate(self.norm(txt), mt[0], mt[1])).view(B, Tt, 3, H, d // H)
        q_i, k_i = (qi[:, :, 0], qi[:, :, 1]) if self.img_qk is None else self.img_qk(qi[:, :, 0], qi[:, :, 1])
        q_t, k_t = (qt[:, :, 0], qt[:, :, 1]) if self.txt_qk is None else self.txt_qk(qt[:, :, 0], qt[:, :, 1])
        o = ops.attention(torch.cat([q_t, q_i], 1), torch.cat([k_t, k_i], 1), torch.cat([qt[:, :, 2], qi[:, :, 2]], 1), causal=False).reshape(B, Tt + Ti, d)
        img = img + mi[2].unsqueeze(1) * self.img_proj(o[:, Tt:])
        img = img + mi[5].unsqueeze(1) * self.img_fc2(F.gelu(self.img_fc1(modulate(self.norm(img), mi[3], mi[4])), approximate="tanh"))
        if not self.pre_only:
            txt = txt + mt[2].unsqueeze(1) * self.txt_proj(o[:, :Tt])
            txt = txt + mt[5].unsqueeze(1) * self.txt_fc2(F.gelu(self.txt_fc1(modulate(self.norm(txt), mt[3], mt[4])), approximate="tanh"))
        return img, txt


@register("sd3")
class SD3Transformer(nn.Module):
    def __init__(self, patch_size: int = 2, input_channels: int = 16, output_channels: Optional[int] = None, emb_features: int = 256,
                 num_heads: int = 4, num_layers: int = 6, mlp_ratio: float = 4.0, text_features: int = 64, pooled_features: int = 32,
                 qk_norm: bool = False):
        super().__init__()
        d = emb_features
        self.patch, self.cout, self.d = patch_size, output_channels or input_channels, d
        self.img_in = Linear(input_channels * patch_size ** 2, d, bias=True)
        self.txt_in = Linear(text_features, d, bias=True)
        self.time_in, self.vector_in = _VectorEmbed(256, d), _VectorEmbed(pooled_features, d)
        self.blocks = nn.ModuleList([_SD3Block(d, num_heads, mlp_ratio, qk_norm, context_pre_only=(i == num_layers - 1)) for i in range(num_layers)])
        self.final_norm = LayerNorm(d, affine=False)
        self.final_mod = Linear(d, 2 * d, bias=True, zero_init=True)
        self.final = Linear(d, self.cout * patch_size ** 2, bias=True, zero_init=True)

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        B, Hh, Ww, C = x.shape
        p = self.patch
        gh, gw = Hh // p, Ww // p
        img = self.img_in(x.reshape(B, gh, p, gw, p, C).permute(0, 1, 3, 2, 4, 5).reshape(B, gh * gw, p * p * C).to(self.img_in.weight.dtype))
        img = img + sincos_2d(gh, gw, self.d, x.device).to(img.dtype)[None]
        text = ctx.get("text")
        if text is None:
            text = torch.zeros(B, 1, self.txt_in.in_features, device=x.device, dtype=img.dtype)
        txt = self.txt_in(text.to(img.dtype))
        c = self.time_in(sinusoidal(temb * 1000.0, 256).to(img.dtype))
        if ctx.get("pooled") is not None:
            c = c + self.vector_in(ctx["pooled"].to(img.dtype))
        for blk in self.blocks:
            img, txt = blk(img, txt, c)
        shift, scale = self.final_mod(F.silu(c)).chunk(2, -1)
        out = self.final(modulate(self.final_norm(img), shift, scale)).float()
        return out.reshape(B, gh, gw, p, p, self.cout).permute(0, 1, 3, 2, 4, 5).reshape(B, Hh, Ww, self.cout)


# ------------------------------------------------------------------------------------------------ Wan
class _WanBlock(nn.Module):
    def __init__(self, d: int, heads: int, ffn: int):
        super().__init__()
        self.heads = heads
        self.modulation = nn.Parameter(torch.zeros(1, 6, d))               # a learned offset on the shared time modulation
        self.norm1, self.norm2 = LayerNorm(d, affine=False), LayerNorm(d, affine=False)
        self.norm3 = LayerNorm(d, affine=True)
        self.qkv, self.o = Linear(d, 3 * d, bias=True), Linear(d, d, bias=True)
        self.self_qk = _QKNorm(d)                                           # Wan normalises queries / keys over the whole width
        self.cq, self.ckv, self.co = Linear(d, d, bias=True), Linear(d, 2 * d, bias=True), Linear(d, d, bias=True)
        self.cross_qk = _QKNorm(d)
        self.fc1, self.fc2 = Linear(d, ffn, bias=True), Linear(ffn, d, bias=True)

    def forward(self, x, e, text, cos, sin):
        B, T, d = x.shape
        H = self.heads
        m = (self.modulation + e).unbind(1)                                  # e: [B, 6, d]
        q, k, v = self.qkv(modulate(self.norm1(x), m[0], m[1])).chunk(3, -1)
        q, k = self.self_qk(q, k)
        q, k = apply_axis_rope(q.view(B, T, H, d // H), cos, sin), apply_axis_rope(k.view(B, T, H, d // H), cos, sin)
        x = x + m[2].unsqueeze(1) * self.o(ops.attention(q, k, v.view(B, T, H, d // H), causal=False).reshape(B, T, d))
        cq = self.cq(self.norm3(x))
        ck, cv = self.ckv(text).chunk(2, -1)
        cq, ck = self.cross_qk(cq, ck)
        Tt = text.shape[1]
        x = x + self.co(ops.attention(cq.view(B, T, H, d // H), ck.view(B, Tt, H, d // H), cv.view(B, Tt, H, d // H), causal=False).reshape(B, T, d))
        return x + m[5].unsqueeze(1) * self.fc2(F.gelu(self.fc1(modulate(self.norm2(x), m[3], m[4])), approximate="tanh"))


@register("wan")
class WanTransformer(nn.Module):
    """Video latents ``[B, F, H, W, C]`` (or images ``[B, H, W, C]``: one frame) -> the same shape."""

    def __init__(self, patch_size: Tuple[int, int, int] = (1, 2, 2), input_channels: int = 16, output_channels: Optional[int] = None,
                 emb_features: int = 256, num_heads: int = 4, num_layers: int = 4, ffn_features: int = 1024, text_features: int = 64,
                 theta: float = 10000.0):
        super().__init__()
        d, hd = emb_features, emb_features // num_heads
        self.patch, self.cout, self.theta = tuple(patch_size), output_channels or input_channels, theta
        self.axes = _default_axes(hd)
        self.patch_in = Linear(input_channels * math.prod(self.patch), d, bias=True)
        self.text_in = _VectorEmbed(text_features, d)
        self.time_in = _VectorEmbed(256, d)
        self.time_proj = Linear(d, 6 * d, bias=True)
        self.blocks = nn.ModuleList([_WanBlock(d, num_heads, ffn_features) for _ in range(num_layers)])
        self.head_norm = LayerNorm(d, affine=False)
        self.head_mod = nn.Parameter(torch.zeros(1, 2, d))
        self.head = Linear(d, self.cout * math.prod(self.patch), bias=True, zero_init=True)

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        image = x.dim() == 4
        if image:
            x = x[:, None]
        B, Fr, Hh, Ww, C = x.shape
        pf, ph, pw = self.patch
        gf, gh, gw = Fr // pf, Hh // ph, Ww // pw
        tok = x.reshape(B, gf, pf, gh, ph, gw, pw, C).permute(0, 1, 3, 5, 2, 4, 6, 7).reshape(B, gf * gh * gw, pf * ph * pw * C)
        h = self.patch_in(tok.to(self.patch_in.weight.dtype))
        text = ctx.get("text")
        if text is None:
            text = torch.zeros(B, 1, self.text_in.fc1.in_features, device=x.device, dtype=h.dtype)
        text = self.text_in(text.to(h.dtype))
        t = self.time_in(sinusoidal(temb * 1000.0, 256).to(h.dtype))
        e = self.time_proj(F.silu(t)).view(B, 6, -1)
        cos, sin = axis_rope(grid_ids(B, gf, gh, gw, x.device), self.axes, self.theta)
        for blk in self.blocks:
            h = blk(h, e, text, cos, sin)
        shift, scale = (self.head_mod + t[:, None]).unbind(1)
        out = self.head(modulate(self.head_norm(h), shift, scale)).float()
        out = out.reshape(B, gf, gh, gw, pf, ph, pw, self.cout).permute(0, 1, 4, 2, 5, 3, 6, 7).reshape(B, Fr, Hh, Ww, self.cout)
        return out[:, 0] if image else out


# ------------------------------------------------------------------------------------------------ EDM2
def mp_silu(x):
    return F.silu(x) / 0.596


def mp_sum(a, b, t: float = 0.5):
    return torch.lerp(a, b, t) / math.sqrt((1 - t) ** 2 + t ** 2)


def mp_cat(a, b, dim: int = 1, t: float = 0.5):
    na, nb = a.shape[dim], b.shape[dim]
    c = math.sqrt((na + nb) / ((1 - t) ** 2 + t ** 2))
    return torch.cat([a * (c / math.sqrt(na) * (1 - t)), b * (c / math.sqrt(nb) * t)], dim)


def pixel_norm(x, dim: int = 1, eps: float = 1e-4):
    n = torch.linalg.vector_norm(x.float(), dim=dim, keepdim=True)
    return (x / (eps + n * math.sqrt(n.numel() / x.numel())).to(x.dtype))


class MPConv(nn.Module):
    """Convolution / linear layer whose weight is re-normalised to unit norm per output channel on every call (and, in training,
    in place: "forced weight normalisation"), so activations keep their magnitude whatever the optimizer does to the weight."""

    def __init__(self, cin: int, cout: int, kernel: Tuple[int, ...] = ()):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(cout, cin, *kernel))

    @staticmethod
    def normalize(w, eps: float = 1e-4):
        n = torch.linalg.vector_norm(w.float(), dim=tuple(range(1, w.dim())), keepdim=True)
        return w / (eps + n * math.sqrt(n.numel() / w.numel())).to(w.dtype)

    def forward(self, x, gain: float = 1.0):
        w = self.weight.float()
        if self.training:
            with torch.no_grad():
                self.weight.copy_(self.normalize(w))
        w = (self.normalize(w) * (gain / math.sqrt(w[0].numel()))).to(x.dtype)
        return x @ w.t() if w.dim() == 2 else F.conv2d(x, w, padding=w.shape[-1] // 2)


class _EDM2Block(nn.Module):
    def __init__(self, cin, cout, cemb, attention: bool, heads_width: int = 64, resample: Optional[str] = None, encoder: bool = True):
        super().__init__()
        self.resample, self.encoder, self.cout = resample, encoder, cout
        self.heads = max(1, cout // heads_width) if attention else 0
        self.emb_gain = nn.Parameter(torch.zeros(()))
        self.conv_res0 = MPConv(cout if encoder else cin, cout, (3, 3))
        self.emb_linear = MPConv(cemb, cout)
        self.conv_res1 = MPConv(cout, cout, (3, 3))
        self.conv_skip = MPConv(cin, cout, (1, 1)) if cin != cout else None
        self.attn_qkv = MPConv(cout, 3 * cout, (1, 1)) if attention else None
        self.attn_proj = MPConv(cout, cout, (1, 1)) if attention else None

    def forward(self, x, emb, res_t: float = 0.3, attn_t: float = 0.3):
        if self.resample == "down":
            x = F.avg_pool2d(x, 2)
        elif self.resample == "up":
            x = F.interpolate(x, scale_factor=2, mode="nearest")
        if self.encoder:
            if self.conv_skip is not None:
                x = self.conv_skip(x)
            x = pixel_norm(x)
        y = self.conv_res0(mp_silu(x))
        c = self.emb_linear(emb, gain=self.emb_gain) + 1
        y = mp_silu(y * c[:, :, None, None].to(y.dtype))
        y = self.conv_res1(y)
        if not self.encoder and self.conv_skip is not None:
            x = self.conv_skip(x)
        x = mp_sum(x, y, res_t)
        if self.heads:
            B, C, Hh, Ww = x.shape
            qkv = pixel_norm(self.attn_qkv(x).reshape(B, self.heads, -1, 3, Hh * Ww), dim=2)
            q, k, v = qkv.unbind(3)
            w = torch.softmax(torch.einsum("bhcq,bhck->bhqk", q.float(), (k / math.sqrt(q.shape[2])).float()), -1).to(v.dtype)
            y = self.attn_proj(torch.einsum("bhqk,bhck->bhcq", w, v).reshape(B, C, Hh, Ww))
            x = mp_sum(x, y, attn_t)
        return x.clamp(-256, 256)


@register("edm2")
class EDM2UNet(nn.Module):
    def __init__(self, input_channels: int = 4, output_channels: Optional[int] = None, features: int = 64, multipliers: Sequence[int] = (1, 2, 3),
                 blocks_per_level: int = 2, attention_levels: Sequence[int] = (1, 2), num_classes: Optional[int] = None, log_variance: bool = True):
        super().__init__()
        cout = output_channels or input_channels
        widths = [features * m for m in multipliers]
        cemb = max(widths)
        self.time_fourier_freqs = nn.Parameter(torch.randn(features) * 2 * math.pi, requires_grad=False)
        self.time_fourier_phases = nn.Parameter(torch.rand(features) * 2 * math.pi, requires_grad=False)
        self.emb_noise = MPConv(features, cemb)
        self.emb_label = MPConv(num_classes, cemb) if num_classes else None
        self.num_classes = num_classes
        self.enc = nn.ModuleList()
        skips = []
        c = input_channels + 1                                  # a constant channel stands in for the bias the layers do not have
        for lvl, w in enumerate(widths):
            if lvl == 0:
                self.enc.append(MPConv(c, w, (3, 3)))
                c = w
            else:
                self.enc.append(_EDM2Block(c, c, cemb, False, resample="down"))
            skips.append(c)
            for _ in range(blocks_per_level):
                self.enc.append(_EDM2Block(c, w, cemb, lvl in attention_levels))
                c = w
                skips.append(c)
        self.dec = nn.ModuleList()
        takes_skip = []
        for lvl in reversed(range(len(widths))):
            w = widths[lvl]
            if lvl == len(widths) - 1:
                self.dec.append(_EDM2Block(c, c, cemb, True, encoder=False))
                self.dec.append(_EDM2Block(c, c, cemb, False, encoder=False))
                takes_skip += [False, False]
            else:
                self.dec.append(_EDM2Block(c, c, cemb, False, resample="up", encoder=False))
                takes_skip.append(False)
            for _ in range(blocks_per_level + 1):
                self.dec.append(_EDM2Block(c + skips.pop(), w, cemb, lvl in attention_levels, encoder=False))
                takes_skip.append(True)
                c = w
        assert not skips
        self.takes_skip = takes_skip
        self.out_conv = MPConv(c, cout, (3, 3))
        self.out_gain = nn.Parameter(torch.zeros(()))
        self.logvar_fourier = nn.Parameter(torch.randn(128) * 2 * math.pi, requires_grad=False) if log_variance else None
        self.logvar_phase = nn.Parameter(torch.rand(128) * 2 * math.pi, requires_grad=False) if log_variance else None
        self.logvar_linear = MPConv(128, 1) if log_variance else None

    def log_variance(self, temb):
        """The learned per-noise-level log-variance EDM2 weights its loss with (``loss / exp(u) + u``)."""
        f = torch.cos(temb.float()[:, None] * self.logvar_fourier + self.logvar_phase) * math.sqrt(2)
        return self.logvar_linear(f)[:, 0]

    def forward(self, x, temb, textcontext=None, train=False, duration=None):
        ctx = _ctx(textcontext)
        h = x.permute(0, 3, 1, 2)
        emb = self.emb_noise(torch.cos(temb.float()[:, None] * self.time_fourier_freqs + self.time_fourier_phases) * math.sqrt(2))
        if self.emb_label is not None and ctx.get("label") is not None:
            onehot = F.one_hot(ctx["label"].long(), self.num_classes).float() * math.sqrt(self.num_classes)
            emb = mp_sum(emb, self.emb_label(onehot), 0.5)
        emb = mp_silu(emb)
        h = torch.cat([h, torch.ones_like(h[:, :1])], 1)
        skips = []
        for layer in self.enc:
            h = layer(h) if isinstance(layer, MPConv) else layer(h, emb)
            skips.append(h)
        for layer, skip in zip(self.dec, self.takes_skip):
            if skip:
                h = mp_cat(h, skips.pop(), 1)
            h = layer(h, emb)
        return self.out_conv(h, gain=self.out_gain).permute(0, 2, 3, 1).float()
