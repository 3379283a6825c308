"""In-context memory: a layer whose inner network's parameters are updated along the sequence by gradient steps on an objective of its
own, and read by every token after its step (Titans, arXiv 2501.00663; TTT, arXiv 2407.04620).  With the views ``k_t, v_t, q_t`` of
the stream and the inner network ``f(W; .)``:

    g_t = grad_W objective(f(W'; k_t), v_t)        taken at the state W' its chunk started from
    S_t = mu_t S_{t-1} - theta_t g_t               momentum (mu = 0 without it)
    W_t = a_t W_{t-1} + S_t                        retention (a = 1 - alpha_t; 1 without it)
    y_t = f(W_t; q_t)                              or f(W'; q_t) when a chunk commits its steps at its end

``theta, mu, alpha`` are per-token, per-head gates computed from the stream; ``W_0`` (the state a document starts from) is the
layer's own meta-learned parameter.  The inner network is a linear map or a two-matrix MLP; its gradients are written out
analytically (``inner_gradients``) so a chunk's are one batched product.  The state (W, S) is kept in fp32.

Two computations give the one function.  ``chunked``: every gradient of a chunk at once, the momentum and the retention across the
chunk as two lower-triangular products of cumulative gate ratios (log space), the readouts one batched product over the per-token
weights - work that is GEMM-shaped and sequential only across chunks.  ``stepped``: token by token, which is the definition and
serves packed rows (a document's first token starts from ``W_0`` with no momentum, chunks counted from there) and streaming
(``state`` carried between calls).

Reference: src/dew/nn/memory.py (``Memory``, ``LinearMemory``), src/dew/nn/continuum.py.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import Linear, RMSNorm, declare

State = Dict[str, object]


def inner_forward(W: Sequence[torch.Tensor], x: torch.Tensor) -> torch.Tensor:
    """``f(W; x)`` for ``x [..., dk]`` and per-position weights ``W[i] [..., a, b]``: one matrix - a linear map; two - ``silu(x W1) W2``."""
    if len(W) == 1:
        return torch.einsum("...k,...kv->...v", x, W[0])
    return torch.einsum("...h,...hv->...v", F.silu(torch.einsum("...k,...kh->...h", x, W[0])), W[1])


def inner_gradients(W: Sequence[torch.Tensor], k: torch.Tensor, v: torch.Tensor, objective: str) -> List[torch.Tensor]:
    """Per-token gradients of the inner objective at ``W``: ``l2`` - half the squared error of ``f(W; k)`` against ``v``; ``dot`` - minus
    their inner product.  ``k [..., dk]``, ``v [..., dv]``, weights broadcast against the leading axes; returns one ``[..., a, b]`` per leaf."""
    if len(W) == 1:
        d = (inner_forward(W, k) - v) if objective == "l2" else -v
        return [k[..., :, None] * d[..., None, :]]
    z = torch.einsum("...k,...kh->...h", k, W[0])
    a = F.silu(z)
    d = (torch.einsum("...h,...hv->...v", a, W[1]) - v) if objective == "l2" else -v
    s = torch.sigmoid(z)
    dz = torch.einsum("...v,...hv->...h", d, W[1]) * (s * (1 + z * (1 - s)))
    return [k[..., :, None] * dz[..., None, :], a[..., :, None] * d[..., None, :]]


def _triangular(log_gate: torch.Tensor) -> torch.Tensor:
    """``[B, C, H]`` log gates -> ``[B, H, C, C]``: entry (t, j) is the product of the gates after j up to t (1 on the diagonal, 0 above)."""
    L = log_gate.cumsum(1).permute(0, 2, 1)
    ratio = L[..., :, None] - L[..., None, :]
    C = L.shape[-1]
    keep = torch.ones(C, C, dtype=torch.bool, device=L.device).tril()
    return torch.where(keep, ratio.masked_fill(~keep, 0.0).exp(), torch.zeros((), device=L.device))


def _wide(p: torch.Tensor) -> torch.Tensor:
    """The state's dtype: at least fp32 (a bf16 state would drop every step below its ulp)."""
    return p.to(torch.promote_types(p.dtype, torch.float32))


class NeuralMemory(nn.Module):
    def __init__(self, features: int, num_heads: int = 4, head_dim: Optional[int] = None, hidden: int = 0, chunk: int = 16, objective: str = "l2",
                 momentum: bool = True, retention: bool = True, commit: bool = False, max_step: float = 1.0, norm_eps: float = 1e-6,
                 dtype=None, device=None):
        super().__init__()
        if objective not in ("l2", "dot"):
            raise ValueError(f"inner objective {objective!r}: known l2 | dot")
        kw = dict(dtype=dtype, device=device)
        self.h, self.d = num_heads, head_dim or features // num_heads
        self.hidden, self.chunk, self.objective, self.commit, self.max_step = hidden, chunk, objective, commit, max_step
        inner = self.h * self.d
        self.qkv_proj = Linear(features, 3 * inner, **kw)
        gates = 1 + int(momentum) + int(retention)
        self.gate_proj = Linear(features, gates * num_heads, bias=True, **kw)
        self.momentum, self.retention = momentum, retention
        shapes = [(self.d, self.d)] if hidden == 0 else [(self.d, hidden), (hidden, self.d)]
        # W_0: what a document's memory starts from, learned by the outer optimiser
        self.initial = nn.ParameterList([declare(nn.Parameter(torch.zeros(num_heads, *s, dtype=torch.float32, device=device)), ("heads", None, None), "memory")
                                         for s in shapes])
        self.norm = RMSNorm(self.d, norm_eps, **kw)
        self.out_gate = Linear(features, inner, **kw)
        self.o_proj = Linear(inner, features, **kw)
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            for p in self.initial:
                p.normal_(0.0, 0.5 / math.sqrt(p.shape[1]), generator=generator) if len(self.initial) > 1 else p.zero_()
            self.gate_proj.bias.zero_()
            if self.retention:                                  # start by keeping nearly everything
                self.gate_proj.bias[-self.h:].fill_(-4.0)

    # ------------------------------------------------------------------ views and gates
    def views(self, x):
        B, T, _ = x.shape
        q, k, v = self.qkv_proj(x).float().view(B, T, 3, self.h, self.d).unbind(2)
        q, k = F.normalize(F.silu(q), dim=-1), F.normalize(F.silu(k), dim=-1)
        g = self.gate_proj(x).float().view(B, T, -1, self.h)
        theta = torch.sigmoid(g[:, :, 0]) * self.max_step
        log_mu = F.logsigmoid(g[:, :, 1]) if self.momentum else None
        log_a = F.logsigmoid(-g[:, :, -1]) if self.retention else None            # a = 1 - alpha
        return q, k, F.silu(v), theta, log_mu, log_a

    def initial_state(self, batch: int) -> State:
        W = [_wide(p)[None].expand(batch, *p.shape).contiguous() for p in self.initial]
        return {"W": W, "S": [torch.zeros_like(w) for w in W], "start": [w.clone() for w in W],
                "count": torch.zeros(batch, dtype=torch.long, device=W[0].device)}

    # ------------------------------------------------------------------ chunk form
    def chunked(self, q, k, v, theta, log_mu, log_a, state: Optional[State] = None) -> Tuple[torch.Tensor, State]:
        B, T = q.shape[:2]
        state = state if state is not None else self.initial_state(B)
        if bool((state["count"] % self.chunk != 0).any()):
            raise ValueError("the chunk form starts on a chunk boundary; carry a mid-chunk state through stepped()")
        W, S = list(state["W"]), list(state["S"])
        outs = []
        for c0 in range(0, T, self.chunk):
            sl = slice(c0, min(T, c0 + self.chunk))
            kc, vc, qc, th = k[:, sl], v[:, sl], q[:, sl], theta[:, sl]
            start = W
            grads = inner_gradients([w[:, None] for w in start], kc, vc, self.objective)           # each [B, C, H, a, b]
            M = _triangular(log_mu[:, sl]) if log_mu is not None else None
            A = _triangular(log_a[:, sl]) if log_a is not None else None
            new_W, new_S, per_token = [], [], []
            for g, w0, s0 in zip(grads, start, S):
                u = -th[..., None, None] * g
                if M is not None:
                    s_all = torch.einsum("bhtj,bjhxy->bthxy", M, u) + M[..., :, 0].permute(0, 2, 1)[..., None, None] * (log_mu[:, sl][:, :1].exp()[..., None, None] * s0[:, None])
                else:
                    s_all = u
                if A is not None:
                    w_all = torch.einsum("bhtj,bjhxy->bthxy", A, s_all) + A[..., :, 0].permute(0, 2, 1)[..., None, None] * (log_a[:, sl][:, :1].exp()[..., None, None] * w0[:, None])
                else:
                    w_all = s_all.cumsum(1) + w0[:, None]
                per_token.append(w_all)
                new_W.append(w_all[:, -1])
                new_S.append(s_all[:, -1])
            outs.append(inner_forward([w[:, None] for w in start] if self.commit else per_token, qc))
            W, S = new_W, new_S
        count = state["count"] + T
        # a call that ends inside a chunk leaves that chunk's start behind, for the stepped form to finish it from
        opened = start if T % self.chunk else [w.clone() for w in W]
        return torch.cat(outs, 1), {"W": W, "S": S, "start": opened, "count": count}

    # ------------------------------------------------------------------ token by token (the definition)
    def stepped(self, q, k, v, theta, log_mu, log_a, state: Optional[State] = None, segment_ids: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, State]:
        B, T = q.shape[:2]
        state = state if state is not None else self.initial_state(B)
        W, S, start, count = list(state["W"]), list(state["S"]), list(state["start"]), state["count"].clone()
        W0 = [_wide(p)[None] for p in self.initial]
        outs = []
        for t in range(T):
            if segment_ids is not None and t > 0:
                first = (segment_ids[:, t] != segment_ids[:, t - 1])[:, None, None, None]
                W = [torch.where(first, w0, w) for w0, w in zip(W0, W)]
                S = [torch.where(first, torch.zeros_like(s), s) for s in S]
                count = torch.where(first[:, 0, 0, 0], torch.zeros_like(count), count)
            opens = (count % self.chunk == 0)[:, None, None, None]
            start = [torch.where(opens, w, s0) for w, s0 in zip(W, start)]
            grads = inner_gradients(start, k[:, t], v[:, t], self.objective)
            th = theta[:, t][..., None, None]
            mu = log_mu[:, t].exp()[..., None, None] if log_mu is not None else 0.0
            a = log_a[:, t].exp()[..., None, None] if log_a is not None else 1.0
            S = [mu * s - th * g for s, g in zip(S, grads)]
            W = [a * w + s for w, s in zip(W, S)]
            outs.append(inner_forward(start if self.commit else W, q[:, t]))
            count = count + 1
        return torch.stack(outs, 1), {"W": W, "S": S, "start": start, "count": count}

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0, state: Optional[State] = None, return_state: bool = False):
        if cache is not None:
            raise NotImplementedError("the memory layer streams through its own state (forward(x, state=..., return_state=True)), not the KV cache")
        B, T, _ = x.shape
        q, k, v, theta, log_mu, log_a = self.views(x)
        mid_chunk = state is not None and bool((state["count"] % self.chunk != 0).any())
        if segment_ids is not None or mid_chunk or T == 1:
            y, new = self.stepped(q, k, v, theta, log_mu, log_a, state, segment_ids)
        else:
            y, new = self.chunked(q, k, v, theta, log_mu, log_a, state)
        y = self.norm(y.to(x.dtype)) * F.silu(self.out_gate(x)).view(B, T, self.h, self.d)
        out = self.o_proj(y.reshape(B, T, self.h * self.d))
        return (out, new) if return_state else out
