"""More of the linear-recurrence family as decoder mixers, each with a step-by-step recurrence (the oracle and the decode path)
and a chunked parallel form for training.

``GatedLinearAttention``  GLA (arXiv 2312.06635): ``S_t = diag(a_t) S_{t-1} + k_t^T v_t``, ``o_t = q_t S_t`` with a per-channel
                          data-dependent gate ``a_t`` in (0, 1) from a low-rank projection; chunked form in log space
``DeltaNet``              the plain delta rule (arXiv 2406.06484): ``S_t = S_{t-1} (I - beta_t k_t k_t^T) + beta_t k_t^T v_t`` -
                          the gated delta rule of this library with the gate held at one
``RWKV7``                 the generalised delta rule of RWKV-7 (arXiv 2503.14456): ``S_t = S_{t-1} (diag(w_t) - k^_t^T (a_t * k^_t)) + v_t^T k_t``,
                          with token-shift mixing, low-rank decay / in-context-rate / value-residual / gate generators and a bonus
                          term; recurrence only (the sequential form), which is what decoding needs and what a reference is

Reference: the linear-recurrence family of src/dew/nn/kernels/templates/recurrence (GLA, RWKV, delta) and src/dew/nn/mixers.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import scan
from .layers import Linear, RMSNorm
from .linear_attention import ShortConv


# ------------------------------------------------------------------------------------------------ gated linear attention
def gla_recurrent(q, k, v, log_a, state=None, scale: Optional[float] = None):
    """``q, k, log_a [B, T, H, dk]``, ``v [B, T, H, dv]`` -> (``o [B, T, H, dv]``, final state ``[B, H, dk, dv]``)."""
    B, T, H, dk = q.shape
    scale = dk ** -0.5 if scale is None else scale
    S = q.new_zeros(B, H, dk, v.shape[-1], dtype=torch.float32) if state is None else state.float()
    out = []
    for t in range(T):
        S = torch.exp(log_a[:, t].float())[..., None] * S + k[:, t].float()[..., None] * v[:, t].float()[..., None, :]
        out.append(torch.einsum("bhk,bhkv->bhv", q[:, t].float() * scale, S))
    return torch.stack(out, 1), S


def gla_chunked(q, k, v, log_a, state=None, scale: Optional[float] = None, chunk: int = 32):
    """The same by chunks: inside a chunk the gates' cumulative sums turn the recurrence into a masked product
    ``(q e^{b}) (k e^{-b})^T`` (``b`` measured from the chunk's start, so its magnitude stays within one chunk's worth of gates);
    across chunks the state is carried."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    pad = (-T) % chunk
    if pad:
        q, k, v, log_a = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v, log_a))
    n = (T + pad) // chunk
    qf, kf, vf, gf = (x.float().reshape(B, n, chunk, H, -1).permute(0, 1, 3, 2, 4) for x in (q, k, v, log_a))        # [B, n, H, C, d]
    b = gf.cumsum(3)                                                     # log of the product of gates from the chunk's start through t
    S = q.new_zeros(B, H, dk, dv, dtype=torch.float32) if state is None else state.float()
    causal = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    outs = []
    for c in range(n):
        bc = b[:, c]                                                     # [B, H, C, dk]
        qs = qf[:, c] * scale
        # between chunks: the carried state, decayed from the chunk's start to t
        inter = torch.einsum("bhck,bhkv->bhcv", qs * torch.exp(bc), S)
        # inside: sum_{s <= t} (q_t e^{b_t - b_s}) . k_s  v_s ; computed per pair in log space to stay bounded
        diff = bc[:, :, :, None, :] - bc[:, :, None, :, :]              # [B, H, C, C, dk], <= 0 where s <= t
        w = torch.exp(diff.masked_fill(~causal[None, None, :, :, None], float("-inf")))
        scores = torch.einsum("bhtk,bhtsk,bhsk->bhts", qs, w, kf[:, c])
        outs.append(inter + torch.einsum("bhts,bhsv->bhtv", scores, vf[:, c]))
        total = bc[:, :, -1]                                             # the whole chunk's decay
        S = torch.exp(total)[..., None] * S + torch.einsum("bhsk,bhsv->bhkv", kf[:, c] * torch.exp(total[:, :, None] - bc), vf[:, c])
    o = torch.stack(outs, 1).permute(0, 1, 3, 2, 4).reshape(B, n * chunk, H, dv)[:, :T]
    return o, S


class GatedLinearAttention(nn.Module):
    def __init__(self, features: int, num_heads: int = 4, expand_k: float = 0.5, expand_v: float = 1.0, gate_rank: int = 16, gate_normalizer: float = 16.0,
                 norm_eps: float = 1e-5, dtype=None, device=None):
        super().__init__()
        self.h = num_heads
        self.key_dim, self.value_dim = int(features * expand_k), int(features * expand_v)
        self.dk, self.dv = self.key_dim // num_heads, self.value_dim // num_heads
        self.q_proj = Linear(features, self.key_dim, dtype=dtype, device=device)
        self.k_proj = Linear(features, self.key_dim, dtype=dtype, device=device)
        self.v_proj = Linear(features, self.value_dim, dtype=dtype, device=device)
        self.g_proj = Linear(features, self.value_dim, dtype=dtype, device=device)
        self.gk_proj = nn.Sequential(Linear(features, gate_rank, dtype=dtype, device=device), Linear(gate_rank, self.key_dim, bias=True, dtype=dtype, device=device))
        self.o_proj = Linear(self.value_dim, features, dtype=dtype, device=device)
        self.norm = RMSNorm(self.dv, norm_eps, dtype=dtype, device=device)
        self.gate_normalizer = gate_normalizer

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0):
        B, T, _ = x.shape
        q = self.q_proj(x).view(B, T, self.h, self.dk)
        k = self.k_proj(x).view(B, T, self.h, self.dk)
        v = self.v_proj(x).view(B, T, self.h, self.dv)
        log_a = F.logsigmoid(self.gk_proj(x).float()).view(B, T, self.h, self.dk) / self.gate_normalizer
        if segment_ids is not None:
            # a document's first token forgets everything before it
            first = torch.cat([torch.ones_like(segment_ids[:, :1], dtype=torch.bool), segment_ids[:, 1:] != segment_ids[:, :-1]], 1)
            log_a = log_a.masked_fill(first[..., None, None], -60.0)
        state = cache.recurrent(layer, B, self) if cache is not None and hasattr(cache, "recurrent") else None
        if state is not None and T == 1:
            o, S = gla_recurrent(q, k, v, log_a, state["S"])
        else:
            o, S = gla_chunked(q, k, v, log_a, state["S"] if state is not None else None)
        if state is not None:
            state["S"].copy_(S)
        o = self.norm(o.to(x.dtype)) * F.silu(self.g_proj(x)).view(B, T, self.h, self.dv)
        return self.o_proj(o.reshape(B, T, self.value_dim))


# ------------------------------------------------------------------------------------------------ delta rule
class DeltaNet(nn.Module):
    def __init__(self, features: int, num_heads: int = 4, head_dim: Optional[int] = None, conv_size: int = 4, norm_eps: float = 1e-5, dtype=None, device=None):
        super().__init__()
        self.h = num_heads
        self.d = head_dim or features // num_heads
        inner = self.h * self.d
        self.qkv_proj = Linear(features, 3 * inner, dtype=dtype, device=device)
        self.beta_proj = Linear(features, num_heads, dtype=dtype, device=device)
        self.conv1d = ShortConv(3 * inner, conv_size, activation=True, dtype=dtype, device=device)
        self.norm = RMSNorm(self.d, norm_eps, dtype=dtype, device=device)
        self.o_proj = Linear(inner, features, dtype=dtype, device=device)

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0):
        B, T, _ = x.shape
        state = cache.recurrent(layer, B, self) if cache is not None and hasattr(cache, "recurrent") else None
        qkv = self.conv1d(self.qkv_proj(x), segment_ids, state["conv"] if state is not None else None)
        q, k, v = (t.reshape(B, T, self.h, self.d) for t in qkv.chunk(3, -1))
        q, k = ops.l2_normalize(q), ops.l2_normalize(k)
        beta = torch.sigmoid(self.beta_proj(x).float())
        g = torch.zeros_like(beta)                                       # no forgetting: the gated delta rule with its gate at one
        if state is not None and T == 1:
            o = scan.gated_delta_rule_step(q[:, 0], k[:, 0], v[:, 0].float(), g[:, 0], beta[:, 0], state["S"])[:, None]
        else:
            o, S = scan.chunk_gated_delta_rule(q, k, v if v.is_cuda else v.float(), g, beta, initial_state=state["S"] if state is not None else None)
            if state is not None:
                state["S"].copy_(S)
        return self.o_proj(self.norm(o.to(x.dtype)).reshape(B, T, self.h * self.d))


# ------------------------------------------------------------------------------------------------ RWKV-7
def rwkv7_recurrent(r, w, k, v, kk, a, state=None):
    """``r, w, k, kk, a [B, T, H, d]`` (``w`` the per-channel decay in (0, 1), ``kk`` the normalised removal key, ``a`` the in-context
    learning rate), ``v [B, T, H, d]`` -> (``o``, final state ``[B, H, d_v, d_k]``): ``S <- S (diag(w) - kk^T (a * kk)) + v^T k``, ``o = S r``."""
    B, T, H, d = r.shape
    S = r.new_zeros(B, H, d, d, dtype=torch.float32) if state is None else state.float()
    out = []
    for t in range(T):
        wt, kt, vt, kkt, at, rt = (x[:, t].float() for x in (w, k, v, kk, a, r))
        S = S * wt[:, :, None, :] - torch.einsum("bhvk,bhk,bhj->bhvj", S, kkt, at * kkt) + vt[..., :, None] * kt[..., None, :]
        out.append(torch.einsum("bhvk,bhk->bhv", S, rt))
    return torch.stack(out, 1), S


class _LoRA(nn.Module):
    def __init__(self, features: int, rank: int, out: int, bias: bool = True, activation=None):
        super().__init__()
        self.a, self.b = nn.Linear(features, rank, bias=False), nn.Linear(rank, out, bias=bias)
        nn.init.zeros_(self.b.weight)
        self.activation = activation

    def forward(self, x):
        h = self.a(x)
        return self.b(self.activation(h) if self.activation is not None else h)


class RWKV7(nn.Module):
    """The time-mix block of RWKV-7.  ``layer_index == 0`` has no value residual to read; later layers mix their value toward the
    first layer's (``cache['v_first']`` / the ``v_first`` argument)."""

    def __init__(self, features: int, num_heads: int = 4, decay_rank: int = 16, rate_rank: int = 16, value_rank: int = 8, gate_rank: int = 32,
                 layer_index: int = 0, norm_eps: float = 64e-5):
        super().__init__()
        self.h, self.d, self.layer_index = num_heads, features // num_heads, layer_index
        C = features
        self.mix = nn.Parameter(torch.full((6, C), 0.5))               # token-shift mixing for r, w, k, v, a, g
        self.r_proj, self.k_proj, self.v_proj, self.o_proj = (nn.Linear(C, C, bias=False) for _ in range(4))
        self.w0 = nn.Parameter(torch.full((C,), -1.0))
        self.w_lora = _LoRA(C, decay_rank, C, bias=False, activation=torch.tanh)
        self.a0 = nn.Parameter(torch.zeros(C))
        self.a_lora = _LoRA(C, rate_rank, C, bias=False)
        if layer_index > 0:
            self.v0 = nn.Parameter(torch.ones(C))
            self.v_lora = _LoRA(C, value_rank, C, bias=False)
        self.g_lora = _LoRA(C, gate_rank, C, bias=False, activation=torch.sigmoid)
        self.k_k = nn.Parameter(torch.full((C,), 0.85))
        self.k_a = nn.Parameter(torch.ones(C))
        self.r_k = nn.Parameter(torch.zeros(num_heads, self.d))
        self.norm = nn.GroupNorm(num_heads, C, eps=norm_eps)

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0, v_first: Optional[torch.Tensor] = None):
        B, T, C = x.shape
        H, d = self.h, self.d
        state = cache.recurrent(layer, B, self) if cache is not None and hasattr(cache, "recurrent") else None
        prev = torch.cat([x.new_zeros(B, 1, C) if state is None or "shift" not in state else state["shift"][:, None].to(x.dtype), x[:, :-1]], 1)
        if segment_ids is not None:
            first = torch.cat([torch.ones_like(segment_ids[:, :1], dtype=torch.bool), segment_ids[:, 1:] != segment_ids[:, :-1]], 1)
            prev = prev.masked_fill(first[..., None], 0.0)
        xr, xw, xk, xv, xa, xg = (x + (prev - x) * self.mix[i] for i in range(6))
        r, k, v = self.r_proj(xr), self.k_proj(xk), self.v_proj(xv)
        w = torch.exp(-math.exp(-0.5) * torch.sigmoid((self.w0 + self.w_lora(xw)).float()))           # decay in (exp(-0.607), 1)
        a = torch.sigmoid((self.a0 + self.a_lora(xa)).float())
        if self.layer_index > 0 and v_first is not None:
            v = v + (v_first - v) * torch.sigmoid(self.v0 + self.v_lora(xv))
        g = self.g_lora(xg)
        kk = F.normalize((k * self.k_k).view(B, T, H, d).float(), dim=-1)
        k = k * (1 + (a.to(k.dtype) - 1) * self.k_a)
        shape = lambda t: t.view(B, T, H, d)
        o, S = rwkv7_recurrent(shape(r), shape(w), shape(k), shape(v), kk, shape(a), state["S"] if state is not None and "S" in state else None)
        if state is not None:
            state["S"] = S
            state["shift"] = x[:, -1].detach()
        o = self.norm(o.reshape(B * T, C).to(x.dtype)).view(B, T, C)
        bonus = ((shape(r) * shape(k) * self.r_k).sum(-1, keepdim=True) * shape(v)).reshape(B, T, C)
        out = self.o_proj((o + bonus) * g)
        return (out, v) if self.layer_index == 0 and v_first is None and getattr(self, "return_v_first", False) else out
