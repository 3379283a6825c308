"""Feed-forward blocks: SwiGLU with one fused gate|up projection, and a GELU MLP (DiT)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import Linear


class SwiGLU(nn.Module):
    """``down(silu(gate(x)) * up(x))``; gate and up share one ``[2F, d]`` weight so the projection is one GEMM
    (the "paired gate|up in one launch" of the reference's GEMM template, src/dew/nn/moe.py:745-770)."""

    def __init__(self, features: int, hidden: int, init_std: Optional[float] = None, activation: str = "silu", dtype=None, device=None):
        super().__init__()
        if activation not in ("silu", "gelu_tanh", "gelu"):
            raise ValueError(f"unknown gate activation {activation!r}; known: silu, gelu_tanh, gelu")
        self.features, self.hidden, self.activation = features, hidden, activation
        self.gate_up_proj = Linear(features, 2 * hidden, axes=("embed", "mlp"), init_std=init_std, dtype=dtype, device=device)
        self.down_proj = Linear(hidden, features, axes=("mlp", "embed"), init_std=init_std, dtype=dtype, device=device)

    def forward(self, x):
        if self.activation == "silu":
            if type(self.gate_up_proj).__name__ == "Linear" and self.gate_up_proj.bias is None:
                return self.down_proj(ops.linear_swiglu(x, self.gate_up_proj.weight))
            return self.down_proj(ops.packed_swiglu(self.gate_up_proj(x)))
        gu = self.gate_up_proj(x)
        g, u = gu.chunk(2, -1)                                    # GeGLU (Gemma): the gate passes through GELU
        return self.down_proj(F.gelu(g, approximate="tanh" if self.activation == "gelu_tanh" else "none") * u)


class GeluMLP(nn.Module):
    def __init__(self, features: int, hidden: int, approximate: str = "tanh", dtype=None, device=None):
        super().__init__()
        self.fc1 = Linear(features, hidden, bias=True, axes=("embed", "mlp"), dtype=dtype, device=device)
        self.fc2 = Linear(hidden, features, bias=True, axes=("mlp", "embed"), dtype=dtype, device=device)
        self.approximate = approximate

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x), approximate=self.approximate))
