"""Condition encoders: the text and vision towers diffusion pipelines and vision-language models bind.

``TransformerEncoder``  pre-LayerNorm blocks with biased projections (the CLIP / SigLIP / ViT / DINOv2 shape): learned positions,
                        GELU or quick-GELU MLPs, optional layer scale, causal or full attention
``VisionTower``         patch embedding (+ class token / register tokens), the encoder, and a head: class token, mean, or SigLIP's
                        attention-pooling probe
``TextTower``           token + position embeddings, the encoder (CLIP's is causal), pooled at the end-of-text token or the last one
``T5Encoder``           T5's encoder stack: relative position buckets shared by all layers, scale-only norms, (gated) GELU / ReLU MLPs

Weights of published checkpoints load through ``dew_b200.interop.encoders``.  Attention runs through ``ops.attention`` (the
flash kernels on a GPU when the shape fits, the reference otherwise); T5's additive position bias takes the explicit-score path.

Reference: src/dew/nn/vision/* (ViT / CLIP / SigLIP encoders), src/dew/interop/text_encoders.py, encoders.py, conditioners.py.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..nn.layers import LayerNorm, Linear


def _act(name: str):
    if name == "quick_gelu":
        return lambda x: x * torch.sigmoid(1.702 * x)
    if name in ("gelu_tanh", "gelu_pytorch_tanh", "gelu_new"):
        return lambda x: F.gelu(x, approximate="tanh")
    if name == "gelu":
        return F.gelu
    if name == "relu":
        return F.relu
    raise ValueError(f"unknown activation {name!r}")


@dataclass
class EncoderConfig:
    features: int = 768
    layers: int = 12
    heads: int = 12
    mlp_features: int = 3072
    activation: str = "gelu"
    norm_eps: float = 1e-5
    layer_scale: bool = False              # DINOv2: a learned per-channel gain on each branch
    causal: bool = False                   # CLIP's text tower


class _Attention(nn.Module):
    def __init__(self, d: int, heads: int, dtype=None, device=None):
        super().__init__()
        self.heads = heads
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (Linear(d, d, bias=True, dtype=dtype, device=device) for _ in range(4))

    def forward(self, x, causal: bool = False, key_mask: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, scale: Optional[float] = None):
        B, S, d = x.shape
        H = self.heads
        q, k, v = (p(x).view(B, S, H, d // H) for p in (self.q_proj, self.k_proj, self.v_proj))
        if key_mask is None and bias is None and scale is None:
            o = ops.attention(q, k, v, causal=causal)
        else:
            s = torch.einsum("bihd,bjhd->bhij", q.float(), k.float()) * (scale if scale is not None else (d // H) ** -0.5)
            if bias is not None:
                s = s + bias
            if causal:
                s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=x.device).triu(1), float("-inf"))
            if key_mask is not None:
                s = s.masked_fill(~key_mask[:, None, None, :].bool(), float("-inf"))
            o = torch.einsum("bhij,bjhd->bihd", torch.softmax(s, -1), v.float()).to(x.dtype)
        return self.out_proj(o.reshape(B, S, d))


class _Block(nn.Module):
    def __init__(self, c: EncoderConfig, dtype=None, device=None):
        super().__init__()
        self.norm1 = LayerNorm(c.features, c.norm_eps, dtype=dtype, device=device)
        self.attn = _Attention(c.features, c.heads, dtype, device)
        self.norm2 = LayerNorm(c.features, c.norm_eps, dtype=dtype, device=device)
        self.fc1 = Linear(c.features, c.mlp_features, bias=True, dtype=dtype, device=device)
        self.fc2 = Linear(c.mlp_features, c.features, bias=True, dtype=dtype, device=device)
        self.act = _act(c.activation)
        self.scale1 = nn.Parameter(torch.ones(c.features, dtype=dtype, device=device)) if c.layer_scale else None
        self.scale2 = nn.Parameter(torch.ones(c.features, dtype=dtype, device=device)) if c.layer_scale else None
        self.causal = c.causal

    def forward(self, x, key_mask=None):
        a = self.attn(self.norm1(x), self.causal, key_mask)
        x = x + (a if self.scale1 is None else a * self.scale1)
        m = self.fc2(self.act(self.fc1(self.norm2(x))))
        return x + (m if self.scale2 is None else m * self.scale2)


class TransformerEncoder(nn.Module):
    def __init__(self, config: EncoderConfig, dtype=None, device=None):
        super().__init__()
        self.config = config
        self.blocks = nn.ModuleList([_Block(config, dtype, device) for _ in range(config.layers)])

    def forward(self, x, key_mask=None, return_layer: Optional[int] = None):
        """``return_layer``: the hidden state after that many blocks (negative counts from the end, as pipelines that take the
        penultimate layer do); None = after the last block."""
        stop = len(self.blocks) if return_layer is None else (return_layer if return_layer >= 0 else len(self.blocks) + 1 + return_layer)
        for blk in self.blocks[:stop]:
            x = blk(x, key_mask)
        return x


class VisionTower(nn.Module):
    """Images ``[B, C, H, W]`` -> (tokens ``[B, N, d]``, pooled ``[B, d]``)."""

    def __init__(self, config: EncoderConfig, image_size: int = 224, patch: int = 16, channels: int = 3, class_token: bool = True,
                 registers: int = 0, pre_norm: bool = False, pool: str = "class", patch_bias: bool = True, norm_tokens: bool = True,
                 dtype=None, device=None):
        super().__init__()
        d = config.features
        self.patch, self.pool, self.norm_tokens = patch, pool, norm_tokens
        self.patch_embed = nn.Conv2d(channels, d, patch, patch, bias=patch_bias, dtype=dtype, device=device)
        n = (image_size // patch) ** 2
        self.class_token = nn.Parameter(torch.zeros(1, 1, d, dtype=dtype, device=device)) if class_token else None
        self.registers = nn.Parameter(torch.zeros(1, registers, d, dtype=dtype, device=device)) if registers else None
        self.position = nn.Parameter(torch.zeros(1, n + int(class_token), d, dtype=dtype, device=device))
        self.pre_norm = LayerNorm(d, config.norm_eps, dtype=dtype, device=device) if pre_norm else None          # CLIP's "pre_layrnorm"
        self.encoder = TransformerEncoder(config, dtype, device)
        self.post_norm = LayerNorm(d, config.norm_eps, dtype=dtype, device=device)
        if pool == "probe":                       # SigLIP: one learned query attends over the tokens, then a residual MLP
            self.probe = nn.Parameter(torch.zeros(1, 1, d, dtype=dtype, device=device))
            self.probe_attn = nn.MultiheadAttention(d, config.heads, batch_first=True, dtype=dtype, device=device)
            self.probe_norm = LayerNorm(d, config.norm_eps, dtype=dtype, device=device)
            self.probe_fc1 = Linear(d, config.mlp_features, bias=True, dtype=dtype, device=device)
            self.probe_fc2 = Linear(config.mlp_features, d, bias=True, dtype=dtype, device=device)
        self.act = _act(config.activation)

    def forward(self, images, return_layer: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        x = self.patch_embed(images).flatten(2).transpose(1, 2)
        if self.class_token is not None:
            x = torch.cat([self.class_token.expand(x.shape[0], -1, -1), x], 1)
        x = x + self.position
        if self.registers is not None:              # registers sit between the class token and the patches, without positions
            lead = 1 if self.class_token is not None else 0
            x = torch.cat([x[:, :lead], self.registers.expand(x.shape[0], -1, -1), x[:, lead:]], 1)
        if self.pre_norm is not None:
            x = self.pre_norm(x)
        x = self.encoder(x, return_layer=return_layer)
        if return_layer is not None:
            return x, x[:, 0]
        if self.pool == "class":
            # CLIP returns the tokens as the last block left them and normalises the class token only; ViT / DINOv2 normalise every
            # token: the pooled output is the same either way
            tokens = self.post_norm(x)
            return (tokens if self.norm_tokens else x), tokens[:, 0]
        tokens = self.post_norm(x)
        if self.pool == "mean":
            return tokens, tokens.mean(1)
        q = self.probe.expand(x.shape[0], -1, -1)
        h = self.probe_attn(q, tokens, tokens, need_weights=False)[0]
        h = h + self.probe_fc2(self.act(self.probe_fc1(self.probe_norm(h))))
        return tokens, h[:, 0]


class TextTower(nn.Module):
    """Token ids ``[B, S]`` -> (states ``[B, S, d]``, pooled ``[B, d]``)."""

    def __init__(self, config: EncoderConfig, vocab_size: int, max_positions: int = 77, pool: str = "eos", eos_token_id: Optional[int] = None,
                 head: bool = False, dtype=None, device=None):
        super().__init__()
        d = config.features
        self.pool, self.eos_token_id = pool, eos_token_id
        self.token = nn.Embedding(vocab_size, d, dtype=dtype, device=device)
        self.position = nn.Embedding(max_positions, d, dtype=dtype, device=device)
        self.encoder = TransformerEncoder(config, dtype, device)
        self.final_norm = LayerNorm(d, config.norm_eps, dtype=dtype, device=device)
        self.head = Linear(d, d, bias=True, dtype=dtype, device=device) if head else None             # SigLIP's text head

    def forward(self, ids, key_mask=None, return_layer: Optional[int] = None):
        S = ids.shape[1]
        x = self.token(ids) + self.position(torch.arange(S, device=ids.device))[None]
        x = self.encoder(x, key_mask, return_layer)
        if return_layer is not None:
            return x, x[:, -1]
        x = self.final_norm(x)
        if self.pool == "eos":
            # CLIP: the state at the end-of-text token (the largest id in the original vocabulary, else the configured one)
            at = ids.argmax(-1) if self.eos_token_id is None else (ids == self.eos_token_id).int().argmax(-1)
            pooled = x[torch.arange(x.shape[0], device=x.device), at]
        else:
            pooled = x[:, -1]
        if self.head is not None:
            pooled = self.head(pooled)
        return x, pooled


# ---------------------------------------------------------------------------------------------------------------- T5
class _T5Norm(nn.Module):
    def __init__(self, d, eps, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)


class _T5Block(nn.Module):
    def __init__(self, d, heads, kv, ff, gated, act, eps, dtype=None, device=None):
        super().__init__()
        self.heads, self.kv = heads, kv
        self.norm1 = _T5Norm(d, eps, dtype, device)
        self.q, self.k, self.v = (Linear(d, heads * kv, dtype=dtype, device=device) for _ in range(3))
        self.o = Linear(heads * kv, d, dtype=dtype, device=device)
        self.norm2 = _T5Norm(d, eps, dtype, device)
        self.wi_0 = Linear(d, ff, dtype=dtype, device=device)
        self.wi_1 = Linear(d, ff, dtype=dtype, device=device) if gated else None
        self.wo = Linear(ff, d, dtype=dtype, device=device)
        self.act = _act(act)

    def forward(self, x, bias, key_mask):
        B, S, d = x.shape
        n = self.norm1(x)
        q, k, v = (p(n).view(B, S, self.heads, self.kv) for p in (self.q, self.k, self.v))
        s = torch.einsum("bihd,bjhd->bhij", q.float(), k.float()) + bias                  # T5 does not scale the scores
        if key_mask is not None:
            s = s.masked_fill(~key_mask[:, None, None, :].bool(), float("-inf"))
        a = torch.einsum("bhij,bjhd->bihd", torch.softmax(s, -1), v.float()).to(x.dtype).reshape(B, S, -1)
        x = x + self.o(a)
        n = self.norm2(x)
        h = self.act(self.wi_0(n))
        if self.wi_1 is not None:
            h = h * self.wi_1(n)
        return x + self.wo(h)


class T5Encoder(nn.Module):
    def __init__(self, vocab_size: int, features: int = 512, layers: int = 6, heads: int = 8, kv: int = 64, ff: int = 1024,
                 gated: bool = True, activation: str = "gelu_new", buckets: int = 32, max_distance: int = 128, eps: float = 1e-6,
                 dtype=None, device=None):
        super().__init__()
        self.buckets, self.max_distance, self.heads = buckets, max_distance, heads
        self.token = nn.Embedding(vocab_size, features, dtype=dtype, device=device)
        self.relative = nn.Embedding(buckets, heads, dtype=dtype, device=device)           # shared by every layer
        self.blocks = nn.ModuleList([_T5Block(features, heads, kv, ff, gated, activation, eps, dtype, device) for _ in range(layers)])
        self.final_norm = _T5Norm(features, eps, dtype, device)

    def position_bias(self, S: int, device) -> torch.Tensor:
        """``[1, heads, S, S]``: the bucketed relative position bias (bidirectional buckets, as the encoder uses)."""
        ctx = torch.arange(S, device=device)[:, None]
        mem = torch.arange(S, device=device)[None, :]
        rel = mem - ctx
        nb = self.buckets // 2
        out = (rel > 0).long() * nb
        rel = rel.abs()
        exact = nb // 2
        large = exact + (torch.log(rel.float().clamp_min(1) / exact) / math.log(self.max_distance / exact) * (nb - exact)).long()
        large = large.clamp_max(nb - 1)
        out = out + torch.where(rel < exact, rel, large)
        return self.relative(out).permute(2, 0, 1)[None].float()

    def forward(self, ids, key_mask=None):
        x = self.token(ids)
        bias = self.position_bias(ids.shape[1], ids.device)
        for blk in self.blocks:
            x = blk(x, bias, key_mask)
        return self.final_norm(x)
