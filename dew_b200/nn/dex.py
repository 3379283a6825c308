"""Differential extension (DEX, arXiv 2505.16333): a learned differential on chosen heads of a pretrained softmax attention layer.  A
chosen head's output ``O_h`` (its attention-weighted values, before the output projection) becomes

    O'_h = O_h - lambda(t) * O_h W_h

with ``W_h`` a learned ``[D, D]`` matrix of the head's own; the other heads are untouched.  ``lambda`` is annealed over the first
``anneal_steps`` optimiser updates from zero to a learned scalar,

    lambda(t) = (1 - a) (t / T) lambda_init + a lambda_learn,     a = min(t / T, 1)

so the model computes its own function when the extension is attached (``lambda(0) = 0``) and the differential enters as it trains.
``lambda_init`` follows the Differential Transformer's depth schedule.  Outside training the layer reads ``lambda_learn``.

``attach_dex(model, heads)`` installs one ``Dex`` per attention layer (``SelfAttention.head_transform``); ``set_progress(model, step)``
tells them the optimiser step; ``head_entropies`` scores heads by the entropy of their attention rows, the statistic the paper picks the
extended half by; ``dex_parameters`` lists what the recipe trains (the extension and the layer's key, value and output projections).

Reference: src/dew/nn/dex.py.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Mapping, Optional, Sequence

import torch
import torch.nn as nn

from .attention_variants import lambda_init
from .layers import declare


class Dex(nn.Module):
    def __init__(self, heads: Sequence[int], head_dim: int, layer: int = 0, anneal_steps: int = 1000, init: Optional[float] = None, dtype=None, device=None):
        super().__init__()
        self.register_buffer("heads", torch.tensor(sorted(heads), dtype=torch.long, device=device), persistent=True)
        self.register_buffer("step", torch.zeros((), dtype=torch.long, device=device), persistent=True)
        self.anneal_steps = max(1, int(anneal_steps))
        self.lambda_init = float(lambda_init(layer) if init is None else init)
        self.weight = declare(nn.Parameter(torch.empty(len(heads), head_dim, head_dim, dtype=dtype, device=device)), ("heads", None, None), "kernel")
        self.lambda_learn = nn.Parameter(torch.tensor(self.lambda_init, dtype=torch.float32, device=device))
        with torch.no_grad():
            self.weight.normal_(0.0, 1.0 / math.sqrt(head_dim))

    def strength(self) -> torch.Tensor:
        if not self.training:
            return self.lambda_learn
        a = min(float(self.step) / self.anneal_steps, 1.0)
        return (1.0 - a) * a * self.lambda_init + a * self.lambda_learn

    def forward(self, o: torch.Tensor) -> torch.Tensor:
        """``o [B, S, H, D]`` -> the same with the chosen heads differenced."""
        chosen = o.index_select(2, self.heads)
        delta = torch.einsum("bshd,hde->bshe", chosen.float(), self.weight.float()) * self.strength()
        return o.index_copy(2, self.heads, (chosen.float() - delta).to(o.dtype))


def attach_dex(model: nn.Module, heads: Mapping[int, Sequence[int]], anneal_steps: int = 1000) -> List[Dex]:
    """Install the extension on the attention layers named by ``heads`` (layer index -> head indices) of a decoder."""
    made = []
    for index, chosen in heads.items():
        mixer = model.layers[index].mixer
        if not hasattr(mixer, "head_transform"):
            raise TypeError(f"layer {index}'s mixer ({type(mixer).__name__}) is not a softmax attention layer")
        p = mixer.o_proj.weight
        mixer.head_transform = Dex(chosen, mixer.head_dim, layer=index, anneal_steps=anneal_steps, dtype=p.dtype, device=p.device)
        made.append(mixer.head_transform)
    return made


def set_progress(model: nn.Module, step: int) -> None:
    for m in model.modules():
        if isinstance(m, Dex):
            m.step.fill_(int(step))


def dex_parameters(model: nn.Module) -> List[nn.Parameter]:
    """What the paper's recipe trains: every extension, and the key / value rows of the packed projection and the output projection of the
    layers that carry one (the packed q | k | v weight is returned whole; mask the query rows' gradient to freeze them)."""
    out: List[nn.Parameter] = []
    for m in model.modules():
        t = getattr(m, "head_transform", None)
        if isinstance(t, Dex):
            out += list(t.parameters()) + [m.qkv_proj.weight, m.o_proj.weight]
    return out


@torch.no_grad()
def head_entropies(q: torch.Tensor, k: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """Mean entropy of each head's attention rows, ``q [B, S, H, D]``, ``k [B, T, Hkv, D]`` -> ``[H]`` (nats)."""
    B, S, H, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    s = torch.einsum("bsgrd,btgd->bgrst", q.float().reshape(B, S, Hkv, H // Hkv, D), k.float()).reshape(B, H, S, T) * D ** -0.5
    if causal:
        mask = torch.arange(T, device=q.device)[None, :] <= torch.arange(S, device=q.device)[:, None] + (T - S)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    return -(p * torch.log(p.clamp_min(1e-30))).sum(-1).mean((0, 2))
