"""A backbone and a decision head, applied as two modules over one parameter tree.

``DecisionModel(backbone, head)(inputs)`` returns ``[B, Q, K]`` option logits with ``-inf`` past each question's options.  The
backbone is anything with ``hidden(tokens, positions, segment_ids) -> [B, L, D]`` (``models.CausalTransformer`` for the
state-first and joint layouts) and, for the readout heads, ``head_weight() -> [V, D]``.  ``BidirectionalBackbone`` is a small
encoder for the marker layout: learned positions, attention inside a row only.

Reference: src/dew/decision/model.py (``DecisionModel``: ``states``, ``readout_logits``, the backbone / head split of the tree).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .head import Head, _Block, _same_row
from .inputs import DecisionInputs


class BidirectionalBackbone(nn.Module):
    def __init__(self, vocab_size: int, features: int = 128, layers: int = 2, heads: Optional[int] = None, max_len: int = 512,
                 dropout: float = 0.0):
        super().__init__()
        self.features = features
        self.embed = nn.Embedding(vocab_size, features)
        self.position = nn.Embedding(max_len, features)
        self.blocks = nn.ModuleList([_Block(features, heads or max(1, features // 64), activation="gelu", dropout=dropout) for _ in range(layers)])
        self.norm = nn.LayerNorm(features)

    def hidden(self, tokens, positions=None, segment_ids=None, cache=None, train: bool = False):
        B, L = tokens.shape
        if positions is None:
            positions = torch.arange(L, device=tokens.device)[None].expand(B, -1)
        if segment_ids is None:
            segment_ids = torch.ones_like(tokens, dtype=torch.int32)
        x = self.embed(tokens) + self.position(positions)
        mask = _same_row(segment_ids, segment_ids)
        for b in self.blocks:
            x = b(x, mask)
        return self.norm(x)

    def head_weight(self):
        return self.embed.weight


def features_of(backbone) -> int:
    cfg = getattr(backbone, "config", None)
    for holder in (backbone, cfg):
        for name in ("features", "emb_features", "hidden_size"):
            v = getattr(holder, name, None) if holder is not None else None
            if isinstance(v, int):
                return v
    raise ValueError("cannot tell the backbone's width: give it a `features` attribute")


class DecisionModel(nn.Module):
    def __init__(self, backbone: nn.Module, head: Head, freeze_backbone: bool = False):
        super().__init__()
        self.backbone, self.head = backbone, head
        if freeze_backbone:
            for p in backbone.parameters():
                p.requires_grad_(False)
        self.frozen = freeze_backbone

    def states(self, inputs: DecisionInputs) -> torch.Tensor:
        if self.frozen:
            with torch.no_grad():
                return self.backbone.hidden(inputs.tokens, inputs.positions, inputs.segment_ids)
        return self.backbone.hidden(inputs.tokens, inputs.positions, inputs.segment_ids)

    def forward(self, inputs: DecisionInputs) -> torch.Tensor:
        states = self.states(inputs)
        table = self.backbone.head_weight() if self.head.reads_table else None
        logits = self.head(states, inputs, table)
        return logits.float().masked_fill(~inputs.options, float("-inf"))

    def record(self):
        return {"head": self.head.record(), "frozen": self.frozen, "features": features_of(self.backbone)}
