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


# ---------------------------------------------------------------------------------------------------------------
# Configuration, variants and adapter files
from dataclasses import dataclass, field  # noqa: E402
from contextlib import contextmanager  # noqa: E402
from typing import Mapping, Sequence, Tuple  # noqa: E402


@dataclass(frozen=True)
class LoRAConfig:
    """Which layers get adapters and of what shape.

    ``targets``       regexes matched against the attribute name of each ``Linear`` (``qkv_proj``, ``down_proj`` ...)
    ``rank`` / ``alpha`` / ``dropout``  the usual; ``rank_pattern`` maps a regex over the module *path* to another rank
    ``rs``            rank-stabilised scaling ``alpha / sqrt(r)`` instead of ``alpha / r`` (rsLoRA)
    ``dora``          weight-decomposed adaptation: the adapted weight's direction comes from ``W + s B A`` and a trainable
                      per-output-row magnitude replaces its row norms (DoRA)
    ``quantize_base`` keep the frozen base weight in a quantised form (``int8`` / ``float8_e4m3fn`` / ``nvfp4``) and
                      de-quantise it for the product: adapter training over a base that costs a quarter to a half of bf16
    """
    targets: Tuple[str, ...] = ("qkv_proj", "o_proj")
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    rank_pattern: Mapping[str, int] = field(default_factory=dict)
    rs: bool = False
    dora: bool = False
    quantize_base: Optional[str] = None
    freeze_rest: bool = True


class DoRALinear(LoRALinear):
    """``y = m * (W + s B A) x / ||W + s B A||_row``: direction from the adapted weight, magnitude ``m`` trainable (initialised
    to the base weight's row norms, so the layer starts as the base)."""

    def __init__(self, base: Linear, rank: int = 8, alpha: float = 16.0, dropout: float = 0.0):
        super().__init__(base, rank, alpha, dropout)
        with torch.no_grad():
            m = base.weight.float().norm(dim=1)
        self.magnitude = declare(nn.Parameter(m.to(base.weight.dtype)), ("mlp",), "scale")

    def forward(self, x):
        if self.merged:
            return self.base(x)
        w = self.base.weight.float() + self.scale * (self.lora_b.float() @ self.lora_a.float())
        norm = w.norm(dim=1).detach()                       # the norm is treated as a constant in the backward (the DoRA paper's choice)
        h = self.dropout(x) if self.dropout is not None else x
        y = self.base(x) + ops.linear(ops.linear(h, self.lora_a), self.lora_b) * self.scale
        if self.base.bias is not None:
            y = y - self.base.bias
        y = y * (self.magnitude.float() / norm).to(y.dtype)
        return y if self.base.bias is None else y + self.base.bias

    def merge(self):
        if not self.merged:
            with torch.no_grad():
                w = self.base.weight.float() + self.scale * (self.lora_b.float() @ self.lora_a.float())
                self._kept = self.base.weight.detach().clone()
                self.base.weight.copy_((w * (self.magnitude.float() / w.norm(dim=1))[:, None]).to(self.base.weight.dtype))
            self.merged = True

    def unmerge(self):
        if self.merged:
            with torch.no_grad():
                self.base.weight.copy_(self._kept)
            self.merged = False


class _QuantizedBase(nn.Module):
    """A frozen ``Linear`` whose weight is held quantised (see ``nn.quantization``) and de-quantised per call."""

    def __init__(self, base: Linear, kind: str):
        super().__init__()
        from .quantization import quantize_weight
        self.kind, self.in_features, self.out_features = kind, base.in_features, base.out_features
        self.dtype = base.weight.dtype
        for k, v in quantize_weight(base.weight.detach(), kind).items():
            self.register_buffer(f"q_{k}", v)
        self.bias = base.bias

    @property
    def weight(self):
        from .quantization import dequantize_weight
        stored = {k[2:]: v for k, v in self._buffers.items() if k.startswith("q_")}
        return dequantize_weight(stored, self.kind, self.dtype)

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


def apply_lora_config(model: nn.Module, cfg: LoRAConfig) -> List[str]:
    """``apply_lora`` driven by a ``LoRAConfig`` (rank patterns, rsLoRA, DoRA, quantised base)."""
    pats = [re.compile(t) for t in cfg.targets]
    wrapped = []
    if cfg.freeze_rest:
        for p in model.parameters():
            p.requires_grad_(False)
    for path, module in list(model.named_modules()):
        for name, child in list(module.named_children()):
            if not (isinstance(child, Linear) and any(p.search(name) for p in pats)):
                continue
            full = f"{path}.{name}" if path else name
            rank = next((r for pat, r in cfg.rank_pattern.items() if re.search(pat, full)), cfg.rank)
            alpha = cfg.alpha * (math.sqrt(rank) if cfg.rs else 1.0)        # alpha / r * sqrt(r) = alpha / sqrt(r)
            cls = DoRALinear if cfg.dora else LoRALinear
            layer = cls(child, rank, alpha, cfg.dropout)
            if cfg.quantize_base:
                layer.base = _QuantizedBase(child, cfg.quantize_base)
            setattr(module, name, layer)
            wrapped.append(full)
    if not wrapped:
        raise ValueError(f"no Linear matches {list(cfg.targets)}; attribute names seen: "
                         f"{sorted({n for _, m in model.named_modules() for n, c in m.named_children() if isinstance(c, Linear)})}")
    return wrapped


@contextmanager
def adapters_disabled(model: nn.Module):
    """Run the base model: every adapter's update is switched off inside the block (the reference policy of DPO-style
    objectives over a LoRA-tuned model needs no second copy of the weights)."""
    layers = [m for m in model.modules() if isinstance(m, LoRALinear)]
    for m in layers:
        m._forward_kept = m.forward
        m.forward = m.base.forward if not m.merged else m._forward_kept
    try:
        yield model
    finally:
        for m in layers:
            m.forward = m._forward_kept
            del m._forward_kept


def load_lora_state(model: nn.Module, state: Mapping[str, torch.Tensor], strict: bool = True) -> None:
    own = {n: p for n, p in model.named_parameters() if ".lora_a" in n or ".lora_b" in n or n.endswith(".magnitude")}
    missing = [k for k in own if k not in state]
    extra = [k for k in state if k not in own]
    if strict and (missing or extra):
        raise KeyError(f"adapter state does not match the model: missing {missing[:4]}, unexpected {extra[:4]}")
    with torch.no_grad():
        for k, p in own.items():
            if k in state:
                p.copy_(state[k].to(p.dtype))


def to_peft_state(model: nn.Module) -> Dict[str, torch.Tensor]:
    """Adapter tensors under the key names the PEFT library writes (``base_model.model.<path>.lora_A.weight`` ...), so an
    adapter trained here loads there."""
    out = {}
    for n, p in model.named_parameters():
        if n.endswith(".lora_a"):
            out[f"base_model.model.{n[:-len('.lora_a')]}.lora_A.weight"] = p.detach().clone()
        elif n.endswith(".lora_b"):
            out[f"base_model.model.{n[:-len('.lora_b')]}.lora_B.weight"] = p.detach().clone()
        elif n.endswith(".magnitude"):
            out[f"base_model.model.{n[:-len('.magnitude')]}.lora_magnitude_vector"] = p.detach().clone()
    return out


def from_peft_state(state: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in state.items():
        k = k[len("base_model.model."):] if k.startswith("base_model.model.") else k
        for src, dst in ((".lora_A.weight", ".lora_a"), (".lora_B.weight", ".lora_b"), (".lora_magnitude_vector", ".magnitude"),
                         (".lora_A.default.weight", ".lora_a"), (".lora_B.default.weight", ".lora_b")):
            if k.endswith(src):
                out[k[:-len(src)] + dst] = v
    return out
