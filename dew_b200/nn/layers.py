"""Basic layers.  Every parameter carries ``logical_axes`` (a tuple of axis names) declared where the parameter is
created; ``dew_b200.parallel.layout`` maps logical axes to mesh axes (reference: docs/design/api.md:268-276,
src/dew/mesh.py:101-146)."""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


def declare(param: nn.Parameter, axes: Sequence[Optional[str]], kind: str = "kernel") -> nn.Parameter:
    param.logical_axes = tuple(axes)
    param.dew_kind = kind
    return param


class Linear(nn.Module):
    """``y = x W^T (+ b)``; ``weight`` is ``[out, in]`` (K-major for the tcgen05 GEMM)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, axes=("embed", "mlp"),
                 init_std: Optional[float] = None, zero_init: bool = False, dtype=None, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        w = torch.empty(out_features, in_features, dtype=dtype, device=device)
        self.weight = declare(nn.Parameter(w), (axes[1], axes[0]), "kernel")
        self.bias = declare(nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)), (axes[1],), "bias") if bias else None
        self.init_std, self.zero_init = init_std, zero_init
        self.reset_parameters()

    def reset_parameters(self, generator: Optional[torch.Generator] = None):
        with torch.no_grad():
            if self.zero_init:
                self.weight.zero_()
            else:
                std = self.init_std if self.init_std is not None else 1.0 / math.sqrt(self.in_features)  # lecun normal
                self.weight.normal_(0.0, std, generator=generator)
            if self.bias is not None:
                self.bias.zero_()

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, features: int, init_std: float = 0.02, dtype=None, device=None):
        super().__init__()
        self.num_embeddings, self.features, self.init_std = num_embeddings, features, init_std
        self.weight = declare(nn.Parameter(torch.empty(num_embeddings, features, dtype=dtype, device=device)),
                              ("vocab", "embed"), "embedding")
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            self.weight.normal_(0.0, self.init_std, generator=generator)

    def forward(self, ids):
        return F.embedding(ids, self.weight)


class RMSNorm(nn.Module):
    def __init__(self, features: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = declare(nn.Parameter(torch.ones(features, dtype=dtype, device=device)), ("norm",), "scale")

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            self.weight.fill_(1.0)

    def forward(self, x, branch=None):
        """With ``branch``: residual-stream form, returns ``(norm(x + branch), x + branch)``."""
        if branch is not None:
            return ops.stream_rms_norm(x, branch, self.weight, self.eps)
        return ops.rms_norm(x, self.weight, self.eps)


class LayerNorm(nn.Module):
    def __init__(self, features: int, eps: float = 1e-6, affine: bool = True, dtype=None, device=None):
        super().__init__()
        self.features, self.eps = features, eps
        self.weight = declare(nn.Parameter(torch.ones(features, dtype=dtype, device=device)), ("norm",), "scale") if affine else None
        self.bias = declare(nn.Parameter(torch.zeros(features, dtype=dtype, device=device)), ("norm",), "bias") if affine else None

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            if self.weight is not None:
                self.weight.fill_(1.0)
                self.bias.zero_()

    def forward(self, x):
        return F.layer_norm(x, (self.features,), self.weight, self.bias, self.eps)


def reset_all(module: nn.Module, seed: int, prefix: str = "") -> None:
    """Re-initialise every sub-module that defines ``reset_parameters`` from one seed (deterministic per module path).
    ``prefix`` is the path of ``module`` inside the model it belongs to, so that initialising a model piece by piece draws
    what initialising it whole would."""
    from ..utils import keys as K
    for name, m in module.named_modules(prefix=prefix):
        fn = getattr(m, "reset_parameters", None)
        if fn is None or any(True for _ in m.children()) and not getattr(m, "_own_reset", False):
            continue
        p = next(m.parameters(recurse=False), None)
        dev = p.device if p is not None else "cpu"
        g = K.generator(K.fold_in(K.key(seed), name), dev)
        try:
            fn(generator=g)
        except TypeError:
            fn()


def sinusoidal(t: torch.Tensor, dim: int, max_period: float = 10000.0, scale: float = 1.0) -> torch.Tensor:
    """Fourier features of a scalar per row: ``[B] -> [B, dim]``."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    args = t.float()[:, None] * scale * freqs[None]
    emb = torch.cat([args.cos(), args.sin()], -1)
    if dim % 2:
        emb = F.pad(emb, (0, 1))
    return emb
