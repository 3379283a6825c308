"""The autoencoders latent-diffusion models are trained in, behind one protocol: ``encode(x) -> z`` and ``decode(z) -> x`` over
channels-last images (videos ``[B, T, H, W, C]``), latents normalised as ``(z - shift) * factor`` (per tensor or per channel).

``AutoencoderKL``   the Stable Diffusion / SDXL / SD3 / FLUX VAE: a convolutional encoder of residual stages with stride-2
                    downsampling (asymmetric padding), a middle block with single-head attention, GroupNorm(32, 1e-6) + SiLU,
                    diagonal-Gaussian moments, optional 1 x 1 quant convolutions; the decoder mirrors it with one more residual
                    block per stage.  Module names follow the published checkpoints' keys, so their state dicts load directly.
``DCAE``            deep-compression autoencoder (32 x - 128 x spatial): every down / up stage carries a non-parametric
                    space-to-channel (channel-to-space) shortcut, so the stage learns a residual on top of a lossless rearrangement
``CausalVideoVAE``  3-D causal convolutions (time padded only toward the past) and per-position channel norms, 8 x spatial and
                    4 x temporal compression: frame 1
                    encodes alone, every 4 following frames to one latent frame, so an image is a one-frame video

Tiling: ``encode`` / ``decode`` take ``tile`` (pixels) to process a large image in overlapping tiles blended linearly across
the overlap, bounding activation memory.

Reference: src/dew/nn/autoencoders/{api,kl,dc_ae,wan,qwen_image}.py (``AutoEncoder`` protocol, ``LatentNormalization``,
``AutoencoderKL``, ``DCAE``, ``WanVAE``), src/dew/interop/autoencoders/pretrained.py.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..utils.registry import register


@dataclass(frozen=True)
class LatentNormalization:
    """``(z - shift) * factor`` and back as ``z / factor + shift``; with ``divides``, ``(z - shift) / factor`` and ``z * factor + shift``.
    ``shift`` / ``factor`` are numbers or per-channel sequences."""
    shift: Union[float, Sequence[float]] = 0.0
    factor: Union[float, Sequence[float]] = 1.0
    divides: bool = False

    def _t(self, v, like: torch.Tensor) -> torch.Tensor:
        return torch.as_tensor(v, dtype=like.dtype, device=like.device)

    def normalize(self, z: torch.Tensor) -> torch.Tensor:
        s, f = self._t(self.shift, z), self._t(self.factor, z)
        return (z - s) / f if self.divides else (z - s) * f

    def restore(self, z: torch.Tensor) -> torch.Tensor:
        s, f = self._t(self.shift, z), self._t(self.factor, z)
        return z * f + s if self.divides else z / f + s


# ------------------------------------------------------------------------------------------------ AutoencoderKL
class ResnetBlock2D(nn.Module):
    def __init__(self, cin: int, cout: int, groups: int = 32, eps: float = 1e-6):
        super().__init__()
        self.norm1 = nn.GroupNorm(groups, cin, eps=eps)
        self.conv1 = nn.Conv2d(cin, cout, 3, padding=1)
        self.norm2 = nn.GroupNorm(groups, cout, eps=eps)
        self.conv2 = nn.Conv2d(cout, cout, 3, padding=1)
        self.conv_shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return h + (x if self.conv_shortcut is None else self.conv_shortcut(x))


class SpatialAttention(nn.Module):
    """Single-head self-attention over the positions of a feature map, with a residual."""

    def __init__(self, channels: int, groups: int = 32, eps: float = 1e-6):
        super().__init__()
        self.group_norm = nn.GroupNorm(groups, channels, eps=eps)
        self.to_q, self.to_k, self.to_v = nn.Linear(channels, channels), nn.Linear(channels, channels), nn.Linear(channels, channels)
        self.to_out = nn.ModuleList([nn.Linear(channels, channels)])

    def forward(self, x):
        B, C, H, W = x.shape
        t = self.group_norm(x).reshape(B, C, H * W).transpose(1, 2)
        o = F.scaled_dot_product_attention(self.to_q(t)[:, None], self.to_k(t)[:, None], self.to_v(t)[:, None])[:, 0]
        return x + self.to_out[0](o).transpose(1, 2).reshape(B, C, H, W)


class _Down(nn.Module):
    def __init__(self, c: int):
        super().__init__()
        self.conv = nn.Conv2d(c, c, 3, stride=2, padding=0)

    def forward(self, x):
        return self.conv(F.pad(x, (0, 1, 0, 1)))           # pad right and bottom only, as the checkpoints were trained


class _Up(nn.Module):
    def __init__(self, c: int):
        super().__init__()
        self.conv = nn.Conv2d(c, c, 3, padding=1)

    def forward(self, x):
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


class _Stage(nn.Module):
    def __init__(self, cin: int, cout: int, layers: int, groups: int, down: bool = False, up: bool = False):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, groups) for i in range(layers)])
        if down:
            self.downsamplers = nn.ModuleList([_Down(cout)])
        if up:
            self.upsamplers = nn.ModuleList([_Up(cout)])

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        if hasattr(self, "downsamplers"):
            x = self.downsamplers[0](x)
        if hasattr(self, "upsamplers"):
            x = self.upsamplers[0](x)
        return x


class _Mid(nn.Module):
    def __init__(self, c: int, groups: int, attention: bool):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(c, c, groups), ResnetBlock2D(c, c, groups)])
        self.attentions = nn.ModuleList([SpatialAttention(c, groups)] if attention else [])

    def forward(self, x):
        x = self.resnets[0](x)
        for a in self.attentions:
            x = a(x)
        return self.resnets[1](x)


class _KLEncoder(nn.Module):
    def __init__(self, cin, latent, widths, layers, groups, attention):
        super().__init__()
        self.conv_in = nn.Conv2d(cin, widths[0], 3, padding=1)
        self.down_blocks = nn.ModuleList([_Stage(widths[max(i - 1, 0)], w, layers, groups, down=i < len(widths) - 1) for i, w in enumerate(widths)])
        self.mid_block = _Mid(widths[-1], groups, attention)
        self.conv_norm_out = nn.GroupNorm(groups, widths[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(widths[-1], 2 * latent, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for b in self.down_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(self.mid_block(x))))


class _KLDecoder(nn.Module):
    def __init__(self, cout, latent, widths, layers, groups, attention):
        super().__init__()
        rev = list(reversed(widths))
        self.conv_in = nn.Conv2d(latent, rev[0], 3, padding=1)
        self.mid_block = _Mid(rev[0], groups, attention)
        self.up_blocks = nn.ModuleList([_Stage(rev[max(i - 1, 0)], w, layers + 1, groups, up=i < len(rev) - 1) for i, w in enumerate(rev)])
        self.conv_norm_out = nn.GroupNorm(groups, rev[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(rev[-1], cout, 3, padding=1)

    def forward(self, z):
        x = self.mid_block(self.conv_in(z))
        for b in self.up_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


def _ramp(n: int, overlap: int, at_start: bool, at_end: bool, device, dtype) -> torch.Tensor:
    """A tile's 1-D blending weight: 1 inside, rising over ``overlap`` entries at a side that meets a neighbour."""
    w = torch.ones(n, device=device, dtype=dtype)
    o = min(overlap, n)
    if o > 0:
        ramp = torch.linspace(0, 1, o + 2, device=device, dtype=dtype)[1:-1]
        if not at_start:
            w[:o] = ramp
        if not at_end:
            w[n - o:] = torch.minimum(w[n - o:], ramp.flip(0))
    return w


def _tiled(fn, x: torch.Tensor, tile: int, overlap: int, scale: float) -> torch.Tensor:
    """Apply ``fn`` (NCHW -> NCHW, resizing by ``scale``) over overlapping tiles of ``x``; the results are summed under feathered
    weights and divided by the weights' sum."""
    B, C, H, W = x.shape
    step = max(1, tile - overlap)
    tops = list(range(0, max(1, H - overlap), step))
    lefts = list(range(0, max(1, W - overlap), step))
    out = wsum = None
    o_out = int(round(overlap * scale))
    for top in tops:
        for left in lefts:
            y = fn(x[:, :, top:top + tile, left:left + tile])
            if out is None:
                out = torch.zeros(B, y.shape[1], int(round(H * scale)), int(round(W * scale)), device=y.device, dtype=y.dtype)
                wsum = torch.zeros(1, 1, out.shape[2], out.shape[3], device=y.device, dtype=y.dtype)
            t0, l0 = int(round(top * scale)), int(round(left * scale))
            h, w = y.shape[2], y.shape[3]
            wy = _ramp(h, o_out, top == tops[0], top + tile >= H, y.device, y.dtype)
            wx = _ramp(w, o_out, left == lefts[0], left + tile >= W, y.device, y.dtype)
            weight = (wy[:, None] * wx[None, :])[None, None]
            out[:, :, t0:t0 + h, l0:l0 + w] += y * weight
            wsum[:, :, t0:t0 + h, l0:l0 + w] += weight
    return out / wsum.clamp_min(1e-8)


@register("autoencoder_kl")
class AutoencoderKL(nn.Module):
    def __init__(self, in_channels: int = 3, latent_channels: int = 4, block_out_channels: Sequence[int] = (128, 256, 512, 512),
                 layers_per_block: int = 2, norm_groups: int = 32, scaling_factor: float = 0.18215, shift_factor: Optional[float] = None,
                 use_quant_conv: bool = True, mid_attention: bool = True):
        super().__init__()
        widths = tuple(block_out_channels)
        self.encoder = _KLEncoder(in_channels, latent_channels, widths, layers_per_block, norm_groups, mid_attention)
        self.decoder = _KLDecoder(in_channels, latent_channels, widths, layers_per_block, norm_groups, mid_attention)
        self.quant_conv = nn.Conv2d(2 * latent_channels, 2 * latent_channels, 1) if use_quant_conv else None
        self.post_quant_conv = nn.Conv2d(latent_channels, latent_channels, 1) if use_quant_conv else None
        self.latent_channels = latent_channels
        self.downsample = 2 ** (len(widths) - 1)
        self.normalization = LatentNormalization(shift_factor or 0.0, scaling_factor)

    # -- presets of the published models' shapes
    @classmethod
    def sd(cls, **kw):
        return cls(latent_channels=4, scaling_factor=0.18215, **kw)

    @classmethod
    def sdxl(cls, **kw):
        return cls(latent_channels=4, scaling_factor=0.13025, **kw)

    @classmethod
    def sd3(cls, **kw):
        return cls(latent_channels=16, scaling_factor=1.5305, shift_factor=0.0609, use_quant_conv=False, **kw)

    @classmethod
    def flux(cls, **kw):
        return cls(latent_channels=16, scaling_factor=0.3611, shift_factor=0.1159, use_quant_conv=False, **kw)

    def _moments(self, x_nchw):
        h = self.encoder(x_nchw)
        return h if self.quant_conv is None else self.quant_conv(h)

    def moments(self, x, tile: Optional[int] = None):
        x = x.permute(0, 3, 1, 2)
        if tile is not None and max(x.shape[2:]) > tile:
            h = _tiled(self._moments, x, tile, tile // 4, 1.0 / self.downsample)
        else:
            h = self._moments(x)
        mean, logvar = h.chunk(2, 1)
        return mean, logvar.clamp(-30.0, 20.0)

    def encode(self, x, sample: bool = False, generator=None, tile: Optional[int] = None):
        mean, logvar = self.moments(x, tile)
        z = mean
        if sample:
            z = mean + torch.exp(0.5 * logvar) * torch.randn(mean.shape, generator=generator, device=mean.device, dtype=mean.dtype)
        return self.normalization.normalize(z.permute(0, 2, 3, 1))

    def _decode(self, z_nchw):
        return self.decoder(z_nchw if self.post_quant_conv is None else self.post_quant_conv(z_nchw))

    def decode(self, z, tile: Optional[int] = None):
        z = self.normalization.restore(z).permute(0, 3, 1, 2)
        t = None if tile is None else tile // self.downsample
        x = _tiled(self._decode, z, t, max(1, t // 4), float(self.downsample)) if t is not None and max(z.shape[2:]) > t else self._decode(z)
        return x.permute(0, 2, 3, 1)

    def loss(self, x, kl_weight: float = 1e-6):
        mean, logvar = self.moments(x)
        z = mean + torch.exp(0.5 * logvar) * torch.randn_like(mean)
        rec = self._decode(z).permute(0, 2, 3, 1)
        kl = 0.5 * (mean ** 2 + logvar.exp() - 1 - logvar).mean()
        return F.mse_loss(rec, x) + kl_weight * kl


# ------------------------------------------------------------------------------------------------ deep-compression autoencoder
def _space_to_channel(x: torch.Tensor, out_channels: int) -> torch.Tensor:
    """Pixel-unshuffle by 2, then average groups of channels down to ``out_channels`` (no parameters)."""
    y = F.pixel_unshuffle(x, 2)
    B, C, H, W = y.shape
    if C % out_channels:
        raise ValueError(f"{C} rearranged channels do not average into {out_channels}")
    return y.reshape(B, out_channels, C // out_channels, H, W).mean(2)


def _channel_to_space(x: torch.Tensor, out_channels: int) -> torch.Tensor:
    """Repeat channels up to ``4 * out_channels``, then pixel-shuffle by 2 (no parameters)."""
    B, C, H, W = x.shape
    need = 4 * out_channels
    if need % C:
        raise ValueError(f"{C} channels do not repeat into {need}")
    return F.pixel_shuffle(x.repeat_interleave(need // C, 1), 2)


class _DCBlock(nn.Module):
    def __init__(self, c: int):
        super().__init__()
        self.conv1, self.conv2 = nn.Conv2d(c, c, 3, padding=1), nn.Conv2d(c, c, 3, padding=1, bias=False)
        self.norm = nn.GroupNorm(1, c, eps=1e-5)                      # (RMS-style norms in the published model; a single-group norm here)

    def forward(self, x):
        return x + self.norm(self.conv2(F.silu(self.conv1(x))))


@register("dc_ae")
class DCAE(nn.Module):
    def __init__(self, in_channels: int = 3, latent_channels: int = 32, widths: Sequence[int] = (64, 128, 256, 256, 512, 512),
                 depths: Sequence[int] = (1, 1, 1, 2, 2, 2), scaling_factor: float = 1.0):
        super().__init__()
        if len(widths) != len(depths):
            raise ValueError("one depth per stage")
        self.widths, self.latent_channels = tuple(widths), latent_channels
        self.downsample = 2 ** (len(widths) - 1)
        self.enc_in = nn.Conv2d(in_channels, widths[0], 3, padding=1)
        self.enc_stages = nn.ModuleList([nn.Sequential(*[_DCBlock(w) for _ in range(d)]) for w, d in zip(widths, depths)])
        if any(w % 4 for w in widths[1:]):
            raise ValueError("stage widths are multiples of 4 (a stage's convolution feeds a pixel-unshuffle)")
        self.enc_down = nn.ModuleList([nn.Conv2d(widths[i], widths[i + 1] // 4, 3, padding=1) for i in range(len(widths) - 1)])
        self.enc_out = nn.Conv2d(widths[-1], latent_channels, 3, padding=1)
        self.dec_in = nn.Conv2d(latent_channels, widths[-1], 3, padding=1)
        self.dec_stages = nn.ModuleList([nn.Sequential(*[_DCBlock(w) for _ in range(d)]) for w, d in zip(reversed(widths), reversed(depths))])
        rev = list(reversed(widths))
        self.dec_up = nn.ModuleList([nn.Conv2d(rev[i], rev[i + 1] * 4, 3, padding=1) for i in range(len(rev) - 1)])
        self.dec_norm = nn.GroupNorm(1, widths[0], eps=1e-5)
        self.dec_out = nn.Conv2d(widths[0], in_channels, 3, padding=1)
        self.normalization = LatentNormalization(0.0, scaling_factor)

    def _encode(self, x):
        x = self.enc_in(x)
        for i, stage in enumerate(self.enc_stages):
            x = stage(x)
            if i < len(self.enc_down):
                x = F.pixel_unshuffle(self.enc_down[i](x), 2) + _space_to_channel(x, self.widths[i + 1])                                    # the stage learns a residual on the rearrangement
        # the latent head has its own shortcut: channel groups of the last features averaged down to the latent's channels
        B, C, H, W = x.shape
        short = x.reshape(B, self.latent_channels, C // self.latent_channels, H, W).mean(2) if C % self.latent_channels == 0 else 0
        return self.enc_out(x) + short

    def _decode(self, z):
        C = self.widths[-1]
        short = z.repeat_interleave(C // z.shape[1], 1) if C % z.shape[1] == 0 else 0
        x = self.dec_in(z) + short
        rev = list(reversed(self.widths))
        for i, stage in enumerate(self.dec_stages):
            x = stage(x)
            if i < len(self.dec_up):
                x = F.pixel_shuffle(self.dec_up[i](x), 2) + _channel_to_space(x, rev[i + 1])
        return self.dec_out(F.silu(self.dec_norm(x)))

    def encode(self, x, sample: bool = False, generator=None, tile=None):
        return self.normalization.normalize(self._encode(x.permute(0, 3, 1, 2)).permute(0, 2, 3, 1))

    def decode(self, z, tile=None):
        return self._decode(self.normalization.restore(z).permute(0, 3, 1, 2)).permute(0, 2, 3, 1)

    def loss(self, x, kl_weight: float = 0.0):
        return F.mse_loss(self.decode(self.encode(x)), x)


# ------------------------------------------------------------------------------------------------ causal video autoencoder
class CausalConv3d(nn.Conv3d):
    """A 3-D convolution whose time axis is padded only toward the past: frame t reads frames <= t."""

    def __init__(self, cin, cout, kernel=3, stride=1):
        k = (kernel,) * 3 if isinstance(kernel, int) else tuple(kernel)
        s = (stride,) * 3 if isinstance(stride, int) else tuple(stride)
        super().__init__(cin, cout, k, s, padding=0)
        self._pad = (k[2] // 2, k[2] // 2, k[1] // 2, k[1] // 2, k[0] - 1, 0)

    def forward(self, x):
        return super().forward(F.pad(x, self._pad))


class _ChannelRMS(nn.Module):
    """RMS normalisation over the channels of each (frame, position) alone: statistics never cross frames, so causality in
    time survives the norm (a GroupNorm over a clip would let frame 1 read every later frame)."""

    def __init__(self, channels: int, eps: float = 1e-6):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones(channels))
        self.eps = eps

    def forward(self, x):
        g = self.gamma.reshape(1, -1, *([1] * (x.dim() - 2)))
        return x * torch.rsqrt(x.float().pow(2).mean(1, keepdim=True) + self.eps).to(x.dtype) * g


class _Res3d(nn.Module):
    def __init__(self, cin, cout, groups=None):
        super().__init__()
        self.norm1, self.conv1 = _ChannelRMS(cin), CausalConv3d(cin, cout)
        self.norm2, self.conv2 = _ChannelRMS(cout), CausalConv3d(cout, cout)
        self.skip = CausalConv3d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv2(F.silu(self.norm2(self.conv1(F.silu(self.norm1(x))))))
        return h + (x if self.skip is None else self.skip(x))


@register("causal_video_vae")
class CausalVideoVAE(nn.Module):
    """``[B, T, H, W, C]`` with ``T = 1 + 4 k`` frames -> latents ``[B, 1 + k, H / 8, W / 8, latent]`` (with the default three spatial
    and two temporal halvings)."""

    def __init__(self, in_channels: int = 3, latent_channels: int = 16, widths: Sequence[int] = (96, 192, 384, 384), temporal: Sequence[bool] = (False, True, True),
                 layers: int = 2, groups: int = 32, shift: Union[float, Sequence[float]] = 0.0, factor: Union[float, Sequence[float]] = 1.0):
        super().__init__()
        self.widths, self.temporal, self.latent_channels = tuple(widths), tuple(temporal), latent_channels
        self.time_factor = 2 ** sum(self.temporal)
        self.downsample = 2 ** (len(widths) - 1)
        self.conv_in = CausalConv3d(in_channels, widths[0])
        self.down = nn.ModuleList()
        for i, w in enumerate(widths):
            cin = widths[max(i - 1, 0)]
            blocks = [_Res3d(cin if j == 0 else w, w, groups) for j in range(layers)]
            self.down.append(nn.ModuleList(blocks))
        self.down_space = nn.ModuleList([nn.Conv3d(w, w, (1, 3, 3), (1, 2, 2), padding=0) for w in widths[:-1]])
        self.down_time = nn.ModuleList([CausalConv3d(w, w, (3, 1, 1), (2, 1, 1)) if t else nn.Identity() for w, t in zip(widths[:-1], self.temporal)])
        self.mid = nn.ModuleList([_Res3d(widths[-1], widths[-1], groups), _Res3d(widths[-1], widths[-1], groups)])
        self.norm_out, self.conv_out = _ChannelRMS(widths[-1]), CausalConv3d(widths[-1], 2 * latent_channels)
        rev = list(reversed(widths))
        self.dec_in = CausalConv3d(latent_channels, rev[0])
        self.dec_mid = nn.ModuleList([_Res3d(rev[0], rev[0], groups), _Res3d(rev[0], rev[0], groups)])
        self.up = nn.ModuleList([nn.ModuleList([_Res3d(rev[max(i - 1, 0)] if j == 0 else w, w, groups) for j in range(layers + 1)]) for i, w in enumerate(rev)])
        self.up_space = nn.ModuleList([nn.Conv3d(w, w, (1, 3, 3), padding=(0, 1, 1)) for w in rev[:-1]])
        self.up_time = nn.ModuleList([CausalConv3d(w, 2 * w, (3, 1, 1)) if t else nn.Identity() for w, t in zip(rev[:-1], reversed(self.temporal))])
        self.dec_norm, self.dec_out = _ChannelRMS(rev[-1]), CausalConv3d(rev[-1], in_channels)
        self.normalization = LatentNormalization(shift, factor)

    def _encode(self, x):                                               # x [B, C, T, H, W]
        x = self.conv_in(x)
        for i, blocks in enumerate(self.down):
            for b in blocks:
                x = b(x)
            if i < len(self.down_space):
                x = self.down_space[i](F.pad(x, (0, 1, 0, 1, 0, 0)))
                if self.temporal[i]:
                    # the first frame stands alone; every following pair of frames becomes one
                    first, rest = x[:, :, :1], x[:, :, 1:]
                    if rest.shape[2]:
                        rest = self.down_time[i](rest)
                    x = torch.cat([first, rest], 2)
        for b in self.mid:
            x = b(x)
        return self.conv_out(F.silu(self.norm_out(x)))

    def _decode(self, z):
        x = self.dec_in(z)
        for b in self.dec_mid:
            x = b(x)
        rev_t = list(reversed(self.temporal))
        for i, blocks in enumerate(self.up):
            for b in blocks:
                x = b(x)
            if i < len(self.up_space):
                if rev_t[i]:
                    first, rest = x[:, :, :1], x[:, :, 1:]
                    if rest.shape[2]:
                        y = self.up_time[i](rest)                       # [B, 2 C, T, H, W] -> interleave into 2 T frames
                        B, C2, T, H, W = y.shape
                        rest = y.reshape(B, 2, C2 // 2, T, H, W).permute(0, 2, 3, 1, 4, 5).reshape(B, C2 // 2, 2 * T, H, W)
                    x = torch.cat([first, rest], 2)
                B, C, T, H, W = x.shape
                x = F.interpolate(x.transpose(1, 2).reshape(B * T, C, H, W), scale_factor=2.0, mode="nearest").reshape(B, T, C, 2 * H, 2 * W).transpose(1, 2)
                x = self.up_space[i](x)
        return self.dec_out(F.silu(self.dec_norm(x)))

    def frames_to_latents(self, frames: int) -> int:
        if (frames - 1) % self.time_factor:
            raise ValueError(f"a clip holds 1 + {self.time_factor} k frames, got {frames}")
        return 1 + (frames - 1) // self.time_factor

    def moments(self, x):
        if x.dim() == 4:
            x = x[:, None]                                              # an image is a one-frame video
        self.frames_to_latents(x.shape[1])
        mean, logvar = self._encode(x.permute(0, 4, 1, 2, 3)).chunk(2, 1)
        return mean, logvar.clamp(-30.0, 20.0)

    def encode(self, x, sample: bool = False, generator=None, tile=None):
        mean, logvar = self.moments(x)
        z = mean + torch.exp(0.5 * logvar) * torch.randn(mean.shape, generator=generator, device=mean.device, dtype=mean.dtype) if sample else mean
        return self.normalization.normalize(z.permute(0, 2, 3, 4, 1))

    def decode(self, z, tile=None):
        return self._decode(self.normalization.restore(z).permute(0, 4, 1, 2, 3)).permute(0, 2, 3, 4, 1)

    def loss(self, x, kl_weight: float = 1e-6):
        mean, logvar = self.moments(x)
        z = mean + torch.exp(0.5 * logvar) * torch.randn_like(mean)
        rec = self._decode(z).permute(0, 2, 3, 4, 1)
        kl = 0.5 * (mean ** 2 + logvar.exp() - 1 - logvar).mean()
        return F.mse_loss(rec, x if x.dim() == 5 else x[:, None]) + kl_weight * kl
