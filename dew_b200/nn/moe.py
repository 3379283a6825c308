"""Mixture-of-experts feed-forward: router, expert-sorted grouped GEMMs, shared experts, aux-loss-free balancing,
capacity, and expert-parallel exchange.

Capability parity: src/dew/nn/moe.py (``Router`` :316-586: softmax / sigmoid scores, top-k, ``norm_topk_prob``, fp32
logits, selection-only ``expert_bias``; ``load_balance_update`` :271; ``expert_dispatch`` :858-930 with
``dispatch='global' | 'exchange'`` and ``capacity_factor``; ``SparseMLP`` :1356-1503 with shared experts and
``shared_gate``), docs/concepts/moe.md:59-106.  Numerics: router logits and every contraction accumulate in fp32.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import grouped as G
from .layers import Linear, declare
from .mlp import SwiGLU


_SELF_GROUP = "self"        # marks a token exchange that spans this rank only, whatever process group exists


class Router(nn.Module):
    use_kernels = True        # False: PyTorch top-k (the comparison arm of the tests)

    def __init__(self, features: int, mix, dtype=None, device=None):
        super().__init__()
        self.mix = mix
        self.weight = declare(nn.Parameter(torch.empty(mix.experts, features, dtype=dtype, device=device)), ("experts", "embed"), "kernel")
        self.register_buffer("expert_bias", torch.zeros(mix.experts, dtype=torch.float32, device=device) if mix.bias else None, persistent=True)
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            self.weight.normal_(0.0, 1.0 / math.sqrt(self.weight.shape[1]), generator=generator)

    def forward(self, x2: torch.Tensor):
        """``x2 [T, d]`` -> (weights [T, k] fp32, expert ids [T, k], scores [T, E] fp32)."""
        mix = self.mix
        logits = F.linear(x2.float(), self.weight.float())
        grouped = getattr(mix, "groups", 1) > 1
        if logits.is_cuda and mix.experts <= 256 and mix.top_k <= 16 and self.use_kernels and not grouped:
            from ..ops.routing import route
            return route(logits, self.expert_bias, mix.top_k, mix.score_function, mix.norm_topk_prob, mix.scaling)
        scores = torch.softmax(logits, -1) if mix.score_function == "softmax" else torch.sigmoid(logits)
        select = scores + self.expert_bias if self.expert_bias is not None else scores     # bias steers selection only
        if grouped:
            # group-limited routing (DeepSeek-V3): a group's score is the sum of its two best experts; experts outside the
            # token's best ``topk_groups`` groups cannot be chosen
            T, E = select.shape
            per = E // mix.groups
            gscore = select.view(T, mix.groups, per).topk(min(2, per), -1).values.sum(-1)
            keep = torch.zeros_like(gscore).scatter_(1, gscore.topk(mix.topk_groups, -1).indices, 1.0).bool()
            select = select.masked_fill(~keep[:, :, None].expand(T, mix.groups, per).reshape(T, E), 0.0)
        _, ids = torch.topk(select, mix.top_k, dim=-1)
        w = scores.gather(-1, ids)
        if mix.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
        return w * mix.scaling, ids, scores


def load_balance_update(bias: torch.Tensor, counts: torch.Tensor, rate: float) -> torch.Tensor:
    """Aux-loss-free balancing: raise the bias of under-loaded experts, lower over-loaded ones by ``rate``."""
    mean = counts.float().mean()
    return bias + rate * torch.sign(mean - counts.float())


def capacity_positions(ids: torch.Tensor, experts: int, capacity: int) -> torch.Tensor:
    """Keep-mask over (token, choice) pairs: a pair is kept if fewer than ``capacity`` earlier pairs chose its expert."""
    flat = ids.reshape(-1)
    onehot = F.one_hot(flat, experts)
    rank = (onehot.cumsum(0) - onehot).gather(1, flat[:, None]).squeeze(1)
    return (rank < capacity).reshape(ids.shape)


class ExpertMLP(nn.Module):
    """E SwiGLU experts with stacked weights: ``gate_up [E, 2F, d]`` and ``down [E, d, F]``."""

    def __init__(self, features: int, hidden: int, experts: int, init_std: Optional[float] = None, dtype=None, device=None):
        super().__init__()
        self.features, self.hidden, self.experts_n = features, hidden, experts
        self.gate_up = declare(nn.Parameter(torch.empty(experts, 2 * hidden, features, dtype=dtype, device=device)), ("experts", "mlp", "embed"), "expert_kernel")
        self.down = declare(nn.Parameter(torch.empty(experts, features, hidden, dtype=dtype, device=device)), ("experts", "embed", "mlp"), "expert_kernel")
        self.init_std = init_std
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            self.gate_up.normal_(0.0, self.init_std or 1.0 / math.sqrt(self.features), generator=generator)
            self.down.normal_(0.0, self.init_std or 1.0 / math.sqrt(self.hidden), generator=generator)

    def param_count_per_expert(self) -> int:
        return 3 * self.features * self.hidden

    def forward(self, xs: torch.Tensor, layout: G.GroupLayout, out: Optional[torch.Tensor] = None, lean: bool = False) -> torch.Tensor:
        """``out`` / ``lean``: honoured by the block-scaled path only (see ``ops.mx.mx_grouped_linear``): the caller checks the
        returned tensor, not the argument."""
        mode = getattr(self, "fp8", False)
        if mode and xs.dtype == torch.bfloat16:
            from ..ops import mx
            if mode != "row" and mx.usable(self.features, 2 * self.hidden) and mx.usable(self.hidden, self.features):
                # block-scaled MXFP8 (1 x 32 blocks, ue8m0 scales applied by the tensor core)
                h = mx.mx_grouped_linear(xs, self.gate_up, layout, None, lean)
                return mx.mx_grouped_linear(ops.packed_swiglu(h), self.down, layout, out, lean)
            from ..ops.fp8 import fp8_grouped_linear            # row / channel scaled e4m3
            h = fp8_grouped_linear(xs, self.gate_up, layout)
            return fp8_grouped_linear(ops.packed_swiglu(h), self.down, layout)
        h = G.grouped_linear(xs, self.gate_up, layout)
        return G.grouped_linear(ops.packed_swiglu(h), self.down, layout)


class SparseMLP(nn.Module):
    use_kernels = True        # False: routing and dispatch / combine by PyTorch index ops (the comparison arm of the tests)

    def __init__(self, features: int, mix, dense_hidden: int, init_std: Optional[float] = None, dtype=None, device=None):
        super().__init__()
        self.mix = mix
        hidden = mix.expert_features or dense_hidden
        self.router = Router(features, mix, dtype=torch.float32, device=device)
        self.experts = ExpertMLP(features, hidden, mix.experts, init_std, dtype=dtype, device=device)
        self.experts.fp8 = mix.fp8            # False | True (block-scaled MXFP8 where the sizes allow) | 'row' (row / channel scaled)
        self.shared = SwiGLU(features, mix.shared_features, init_std, dtype=dtype, device=device) if mix.shared_features else None
        self.shared_gate = Linear(features, 1, axes=("embed", None), dtype=dtype, device=device) if (mix.shared_gate and mix.shared_features) else None
        self.last: Dict[str, Any] = {}
        self.keep_router_outputs = False   # set by objectives.routing.ExpertBalance: keep per-token scores / choices / log partitions
        self.ep = None            # set by dew_b200.parallel.ep.ExpertParallel when the experts are sharded over ranks
        self._exchange = None     # this layer's single-rank token exchange (created on first use on a GPU)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        mix = self.mix
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        T = x2.shape[0]
        self.router.use_kernels = self.use_kernels
        w, ids, scores = self.router(x2)
        if mix.capacity_factor is not None:
            cap = max(int(math.ceil(T * mix.top_k / mix.experts * mix.capacity_factor)), int(mix.capacity_factor))
            keep = capacity_positions(ids, mix.experts, cap)
            w = w * keep
        counts = torch.bincount(ids.reshape(-1), minlength=mix.experts)
        # balance statistics (Switch-style auxiliary loss value, also the signal for the bias update)
        frac = counts.float() / max(1, T * mix.top_k)
        self.last = {"counts": counts, "balance_loss": mix.experts * (frac * scores.mean(0)).sum()}
        if self.keep_router_outputs:
            self.last.update(scores=scores, ids=ids, shape=(int(math.prod(shape[:-2])) if len(shape) > 2 else 1, int(shape[-2])),
                             log_z=torch.logsumexp(F.linear(x2.float(), self.router.weight.float()), -1))
        if self.ep is not None:
            y = self.ep.dispatch_compute_combine(self, x2, w, ids)
        elif x2.is_cuda and x2.dtype == torch.bfloat16 and mix.experts <= 256 and mix.top_k <= 16 and self.use_kernels:
            # one rank: the same device-planned dispatch / combine kernels, with this rank as its own only peer
            from ..parallel.ep import TokenExchange, exchange_experts
            if self._exchange is None:
                self._exchange = TokenExchange(mix.experts, _SELF_GROUP)
            y = exchange_experts(self._exchange, self.experts, x2, w, ids)
        else:
            layout = G.group_layout(ids, mix.experts)
            xs = G.permute(x2, layout, mix.top_k)
            ys = self.experts(xs, layout)
            y = G.combine(ys, layout, w.to(x2.dtype) if x2.dtype != torch.float32 else w, T)
        if self.shared is not None:
            s = self.shared(x2)
            if self.shared_gate is not None:
                s = s * torch.sigmoid(self.shared_gate(x2).float()).to(s.dtype)
            y = y + s
        return y.reshape(shape)
