"""Block attention residuals: the residual stream as a softmax over depth.  The layers are cut into blocks of ``block_size``; each block's
output sum is kept, and every sub-layer reads not the running sum but a softmax mixture of the finished blocks and the current partial
sum, weighted by one learned pseudo-query per read site:

    v      = [block_0, ..., block_{n-1}, partial]          # [B, S, n + 1, D]
    k      = v / sqrt(mean(v^2) + eps)                     # fp32, per source
    scores = k @ (scale * kernel)                          # [B, S, n + 1]
    h      = softmax(scores) @ v

A zero kernel averages the sources.  Layer ``i`` opens a block when ``i % block_size == 0``: after its mixer has read its input, the
partial it received becomes a finished block and the partial restarts from the mixer's output.  Layer 0 reads the embeddings as block
0, and after the last layer a model-level site mixes all blocks with the final partial before the final norm.

``DepthMix`` is one read site; ``depth_residual_forward`` runs a decoder's layers this way (``TransformerConfig.depth_residual_block``).

Reference: src/dew/nn/attention_residuals.py.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.nn as nn

from .layers import declare


class DepthMix(nn.Module):
    def __init__(self, features: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.scale = declare(nn.Parameter(torch.ones(features, dtype=dtype, device=device)), ("norm",), "scale")
        self.kernel = declare(nn.Parameter(torch.zeros(features, dtype=dtype, device=device)), ("embed",), "kernel")

    def forward(self, sources: Sequence[torch.Tensor]) -> torch.Tensor:
        if len(sources) == 1:
            return sources[0]
        v = torch.stack(list(sources), 2).float()                                     # [B, S, n, D]
        k = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        scores = k @ (self.scale.float() * self.kernel.float())                       # [B, S, n]
        return (torch.softmax(scores, -1).unsqueeze(-1) * v).sum(2).to(sources[0].dtype)


class DepthResidualSites(nn.Module):
    """The read sites of a decoder of ``layers`` layers: one in front of every mixer, one in front of every MLP, one before the final norm."""

    def __init__(self, layers: int, features: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.mixer = nn.ModuleList(DepthMix(features, eps, dtype, device) for _ in range(layers))
        self.mlp = nn.ModuleList(DepthMix(features, eps, dtype, device) for _ in range(layers))
        self.out = DepthMix(features, eps, dtype, device)


def depth_residual_forward(layers, sites: DepthResidualSites, h: torch.Tensor, block_size: int, call_mixer, call_mlp) -> torch.Tensor:
    """``call_mixer(layer, x)`` / ``call_mlp(layer, x)`` run a layer's normalised sub-layers on the input the site read; returns what the
    final norm reads."""
    blocks: List[torch.Tensor] = []
    partial = h
    for i, layer in enumerate(layers):
        a = call_mixer(layer, sites.mixer[i](blocks + [partial]))
        if i % block_size == 0:
            blocks.append(partial)
            partial = a
        else:
            partial = partial + a
        if layer.mlp is not None:
            partial = partial + call_mlp(layer, sites.mlp[i](blocks + [partial]))
    return sites.out(blocks + [partial])
