"""GPT-OSS's sparse feed-forward: a biased router that takes the top-k logits and softmaxes those alone, and biased experts whose
activation is a clamped GLU - ``(up + 1) * gate * sigmoid(1.702 gate)`` with the gate clamped above at 7 and the linear half to
``[-7, 7]``.  The published checkpoints interleave the gate and the linear half column by column (``gate_up[..., ::2]`` /
``[..., 1::2]``) and store the matrices input-major; here the experts keep this library's stacked K-major layout (``gate_up [E, 2F, d]`` with
the gate rows first, ``down [E, d, F]``) so the grouped tcgen05 GEMM serves them, and ``interop.families`` converts on load and export.

Tokens are sorted by expert into the aligned padded buffer (``ops.grouped``); both projections are grouped GEMMs; the biases and the
activation are element-wise passes between them.

Reference: src/dew/nn/gpt_oss.py, src/dew/interop/families/gpt_oss.py.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import grouped as G
from .layers import declare

ALPHA, LIMIT = 1.702, 7.0


def clamped_glu(gate_up: torch.Tensor, limit: float = LIMIT, alpha: float = ALPHA) -> torch.Tensor:
    """``[..., 2F]`` holding the gate half then the linear half -> ``[..., F]``."""
    Fh = gate_up.shape[-1] // 2
    gate, up = gate_up[..., :Fh].float().clamp(max=limit), gate_up[..., Fh:].float().clamp(-limit, limit)
    return ((up + 1.0) * gate * torch.sigmoid(alpha * gate)).to(gate_up.dtype)


class TopLogitRouter(nn.Module):
    """``softmax`` over the ``k`` largest biased logits of each token (not over all experts)."""

    def __init__(self, features: int, experts: int, top_k: int, device=None):
        super().__init__()
        self.top_k = top_k
        self.weight = declare(nn.Parameter(torch.empty(experts, features, dtype=torch.float32, device=device)), ("experts", "embed"), "kernel")
        self.bias = declare(nn.Parameter(torch.zeros(experts, dtype=torch.float32, device=device)), ("experts",), "bias")
        self.expert_bias = None                       # (no aux-loss-free balancing bias: the decoder's balance step skips this layer)
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            self.weight.normal_(0.0, 1.0 / math.sqrt(self.weight.shape[1]), generator=generator)
            self.bias.zero_()

    def forward(self, x2: torch.Tensor):
        logits = F.linear(x2.float(), self.weight, self.bias)
        top, ids = torch.topk(logits, self.top_k, dim=-1)
        return torch.softmax(top, -1), ids, logits


class ClampedGluExperts(nn.Module):
    """E biased experts with stacked weights: ``gate_up [E, 2F, d]`` (gate rows first), ``down [E, d, F]``."""

    def __init__(self, features: int, hidden: int, experts: int, init_std: Optional[float] = None, dtype=None, device=None):
        super().__init__()
        self.features, self.hidden, self.init_std = features, hidden, init_std
        kw = dict(dtype=dtype, device=device)
        self.gate_up = declare(nn.Parameter(torch.empty(experts, 2 * hidden, features, **kw)), ("experts", "mlp", "embed"), "expert_kernel")
        self.gate_up_bias = declare(nn.Parameter(torch.zeros(experts, 2 * hidden, **kw)), ("experts", "mlp"), "bias")
        self.down = declare(nn.Parameter(torch.empty(experts, features, hidden, **kw)), ("experts", "embed", "mlp"), "expert_kernel")
        self.down_bias = declare(nn.Parameter(torch.zeros(experts, features, **kw)), ("experts", "embed"), "bias")
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            self.gate_up.normal_(0.0, self.init_std or 1.0 / math.sqrt(self.features), generator=generator)
            self.down.normal_(0.0, self.init_std or 1.0 / math.sqrt(self.hidden), generator=generator)
            self.gate_up_bias.zero_()
            self.down_bias.zero_()

    def param_count_per_expert(self) -> int:
        return 3 * self.features * self.hidden + 2 * self.hidden + self.features

    def forward(self, xs: torch.Tensor, layout: G.GroupLayout) -> torch.Tensor:
        E = self.gate_up.shape[0]
        # the expert that owns each row of the padded buffer (rows of padding take a neighbour's bias and are never combined)
        owner = torch.searchsorted(layout.offsets[1:].long().contiguous(), torch.arange(xs.shape[0], device=xs.device), right=True).clamp_max(E - 1)
        h = G.grouped_linear(xs, self.gate_up, layout) + self.gate_up_bias[owner]
        return G.grouped_linear(clamped_glu(h), self.down, layout) + self.down_bias[owner]


class ClampedGluMoE(nn.Module):
    """Stands where ``SparseMLP`` does when ``Mixture(style='clamped_glu')``."""

    def __init__(self, features: int, mix, dense_hidden: int, init_std: Optional[float] = None, dtype=None, device=None):
        super().__init__()
        self.mix = mix
        self.router = TopLogitRouter(features, mix.experts, mix.top_k, device=device)
        self.experts = ClampedGluExperts(features, mix.expert_features or dense_hidden, mix.experts, init_std, dtype=dtype, device=device)
        self.last: Dict[str, Any] = {}
        self.shared = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        mix, shape = self.mix, x.shape
        x2 = x.reshape(-1, shape[-1])
        T = x2.shape[0]
        w, ids, logits = self.router(x2)
        counts = torch.bincount(ids.reshape(-1), minlength=mix.experts)
        self.last = {"counts": counts, "balance_loss": mix.experts * (counts.float() / max(1, T * mix.top_k) * torch.softmax(logits, -1).mean(0)).sum()}
        layout = G.group_layout(ids, mix.experts)
        ys = self.experts(G.permute(x2, layout, mix.top_k), layout)
        y = G.combine(ys, layout, w.to(x2.dtype) if x2.dtype != torch.float32 else w, T)
        return y.reshape(shape)
