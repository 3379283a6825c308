"""LoRA adapters: wrap chosen ``Linear`` layers with a frozen base weight plus a trainable low-rank update
``W + (alpha / r) B A``; merge / unmerge; adapter-only state for checkpoints (reference: src/dew/lora.py)."""
from __future__ import annotations

import math
import re
from typing import Dict, Iterable, List, Optional

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, declare


class LoRALinear(nn.Module):
    def __init__(self, base: Linear, rank: int = 8, alpha: float = 16.0, dropout: float = 0.0):
        super().__init__()
        self.base, self.rank, self.scale = base, rank, alpha / rank
        self.base.weight.requires_grad_(False)
        dt, dev = base.weight.dtype, base.weight.device
        self.lora_a = declare(nn.Parameter(torch.empty(rank, base.in_features, dtype=dt, device=dev)), ("lora", "embed"), "kernel")
        self.lora_b = declare(nn.Parameter(torch.zeros(base.out_features, rank, dtype=dt, device=dev)), ("mlp", "lora"), "kernel")
        self.dropout = nn.Dropout(dropout) if dropout else None
        self.merged = False
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            self.lora_a.normal_(0.0, 1.0 / math.sqrt(self.base.in_features), generator=generator)
            self.lora_b.zero_()

    @property
    def weight(self):
        return self.base.weight

    @property
    def in_features(self):
        return self.base.in_features

    @property
    def out_features(self):
        return self.base.out_features

    def forward(self, x):
        y = self.base(x)
        if self.merged:
            return y
        h = self.dropout(x) if self.dropout is not None else x
        return y + ops.linear(ops.linear(h, self.lora_a), self.lora_b) * self.scale

    def merge(self):
        if not self.merged:
            with torch.no_grad():
                self.base.weight.add_((self.lora_b.float() @ self.lora_a.float() * self.scale).to(self.base.weight.dtype))
            self.merged = True

    def unmerge(self):
        if self.merged:
            with torch.no_grad():
                self.base.weight.sub_((self.lora_b.float() @ self.lora_a.float() * self.scale).to(self.base.weight.dtype))
            self.merged = False


def apply_lora(model: nn.Module, targets: Iterable[str] = ("qkv_proj", "o_proj"), rank: int = 8, alpha: float = 16.0,
               dropout: float = 0.0, freeze_rest: bool = True) -> List[str]:
    """Replace every ``Linear`` whose attribute name matches one of ``targets`` (regexes); returns the wrapped paths."""
    pats = [re.compile(t) for t in targets]
    wrapped = []
    if freeze_rest:
        for p in model.parameters():
            p.requires_grad_(False)
    for path, module in list(model.named_modules()):
        for name, child in list(module.named_children()):
            if isinstance(child, Linear) and any(p.search(name) for p in pats):
                setattr(module, name, LoRALinear(child, rank, alpha, dropout))
                wrapped.append(f"{path}.{name}" if path else name)
    return wrapped


def lora_state(model: nn.Module) -> Dict[str, torch.Tensor]:
    return {n: p.detach().clone() for n, p in model.named_parameters() if ".lora_a" in n or ".lora_b" in n}


def merge_all(model: nn.Module) -> None:
    for m in model.modules():
        if isinstance(m, LoRALinear):
            m.merge()
