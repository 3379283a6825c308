"""Attention variants beside the standard mixer, each over the library's attention op where its arithmetic allows and in plain
tensor arithmetic where it needs a bias or a selection the kernels do not take.

``DifferentialAttention``   ``softmax(Q1 K1^T) V - lambda softmax(Q2 K2^T) V`` per head (arXiv 2410.05258): two calls of the attention op
                            over one value stream, ``lambda`` re-parameterised as in the paper, a per-head RMS norm and the
                            ``(1 - lambda_init)`` gain
``ForgettingAttention``     the Forgetting Transformer (FoX, arXiv 2503.02130): a per-head forget gate ``f = sigmoid(W x)``; each logit
                            gains ``G_i - G_j`` with ``G`` the cumulative log of the gates, so a key fades with the gates between it
                            and the query
``moba_selection`` / ``block_sparse_attention``   block-selected attention: each query reads the key blocks it selects (MoBA's gate
                            over block-mean keys: its own block always, the best ``top_k - 1`` earlier ones)
``indexed_sparse_attention`` / ``LightningIndexer``   DeepSeek sparse attention's shape: a small indexer scores every visible key
                            (``sum_h w_h relu(q_h . k)``), the top ``k`` keys per query are attended
``ValueExperts``            routed value experts (MoVA): the value projection is a mixture of ``experts`` projections, ``top_k`` per token

Reference: src/dew/nn/differential_attention.py, forgetting_attention.py, block_sparse.py, sparse_selection.py, value_experts.py.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import Linear, RMSNorm


def _causal_mask(S: int, T: int, device) -> torch.Tensor:
    return torch.arange(T, device=device)[None, :] <= (torch.arange(S, device=device)[:, None] + (T - S))


def biased_attention(q, k, v, bias: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """``softmax(scale q k^T + bias) v`` over ``[B, S, H, D]`` queries and ``[B, T, Hkv, D]`` keys / values (grouped heads), with a
    boolean ``mask`` of visible pairs broadcastable to ``[B, H, S, T]``.  A query that sees no key returns zeros."""
    B, S, H, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    scale = D ** -0.5 if scale is None else scale
    s = torch.einsum("bsgrd,btgd->bgrst", q.float().reshape(B, S, Hkv, g, D), k.float()) * scale
    s = s.reshape(B, H, S, T)
    if bias is not None:
        s = s + bias
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.einsum("bgrst,btgd->bsgrd", p.reshape(B, Hkv, g, S, T), v.float())
    return o.reshape(B, S, H, v.shape[-1]).to(q.dtype)


# ------------------------------------------------------------------------------------------------ differential attention
def lambda_init(layer: int) -> float:
    """The paper's schedule of the initial lambda over depth (layer counted from 0)."""
    return 0.8 - 0.6 * math.exp(-0.3 * layer)


class DifferentialAttention(nn.Module):
    def __init__(self, features: int, num_heads: int, num_kv_heads: Optional[int] = None, layer: int = 0, causal: bool = True, norm_eps: float = 1e-5,
                 dtype=None, device=None):
        super().__init__()
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads or num_heads
        self.head_dim = features // num_heads // 2                     # each head holds two query / key halves of this width
        self.causal = causal
        d = self.head_dim
        self.q_proj = Linear(features, 2 * num_heads * d, dtype=dtype, device=device)
        self.k_proj = Linear(features, 2 * self.num_kv_heads * d, dtype=dtype, device=device)
        self.v_proj = Linear(features, self.num_kv_heads * 2 * d, dtype=dtype, device=device)
        self.o_proj = Linear(num_heads * 2 * d, features, dtype=dtype, device=device)
        self.lambda_init = lambda_init(layer)
        self.lambda_q1, self.lambda_k1 = nn.Parameter(torch.randn(d) * 0.1), nn.Parameter(torch.randn(d) * 0.1)
        self.lambda_q2, self.lambda_k2 = nn.Parameter(torch.randn(d) * 0.1), nn.Parameter(torch.randn(d) * 0.1)
        self.subln = RMSNorm(2 * d, norm_eps, dtype=dtype, device=device)
        self.rope_theta = 10000.0
        self._rope = None

    def _tables(self, length: int, device):
        """Rotary tables of this module's own half-width heads (the decoder's tables are built for its full head width)."""
        if self._rope is None or self._rope[0].shape[0] < length or self._rope[0].device != device:
            self._rope = ops.rope_tables(length, self.head_dim, self.rope_theta, device)
        return self._rope

    def lam(self) -> torch.Tensor:
        return torch.exp((self.lambda_q1 * self.lambda_k1).sum().float()) - torch.exp((self.lambda_q2 * self.lambda_k2).sum().float()) + self.lambda_init

    def forward(self, x, cos=None, sin=None, positions=None, segment_ids=None, cache=None, layer=None):
        B, S, _ = x.shape
        H, Hkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        q = self.q_proj(x).view(B, S, 2 * H, d)
        k = self.k_proj(x).view(B, S, 2 * Hkv, d)
        v = self.v_proj(x).view(B, S, Hkv, 2 * d)
        if cos is not None:
            c, s_ = self._tables(cos.shape[0], x.device)
            q, k = ops.rope(q, c, s_, positions), ops.rope(k, c, s_, positions)
        # the two maps of head h are query heads 2h and 2h + 1 (and key heads 2g, 2g + 1): split them into two attention calls
        q1, q2 = q[:, :, 0::2], q[:, :, 1::2]
        k1, k2 = k[:, :, 0::2], k[:, :, 1::2]
        mask = _causal_mask(S, S, x.device)[None, None] if self.causal else None
        if segment_ids is not None:
            same = (segment_ids[:, :, None] == segment_ids[:, None, :])[:, None]
            mask = same if mask is None else mask & same
        a1 = biased_attention(q1, k1, v, mask=mask)
        a2 = biased_attention(q2, k2, v, mask=mask)
        out = self.subln(a1 - self.lam().to(a1.dtype) * a2) * (1 - self.lambda_init)
        return self.o_proj(out.reshape(B, S, H * 2 * d))


# ------------------------------------------------------------------------------------------------ forgetting attention
def forgetting_bias(log_gates: torch.Tensor) -> torch.Tensor:
    """``log_gates [B, S, H]`` (log of each token's forget gate) -> the logit bias ``[B, H, S, S]``: ``G_i - G_j`` with ``G`` the
    cumulative sum, i.e. the sum of the log gates of tokens ``j + 1 .. i``."""
    G = log_gates.float().cumsum(1).permute(0, 2, 1)
    return G[:, :, :, None] - G[:, :, None, :]


class ForgettingAttention(nn.Module):
    def __init__(self, features: int, num_heads: int, num_kv_heads: Optional[int] = None, head_dim: Optional[int] = None, qk_norm: bool = True,
                 dtype=None, device=None):
        super().__init__()
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads or num_heads
        self.head_dim = head_dim or features // num_heads
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        self.qkv_proj = Linear(features, (H + 2 * Hkv) * D, dtype=dtype, device=device)
        self.gate_proj = Linear(features, H, bias=True, dtype=dtype, device=device)
        self.o_proj = Linear(H * D, features, dtype=dtype, device=device)
        self.q_norm = RMSNorm(D, dtype=dtype, device=device) if qk_norm else None
        self.k_norm = RMSNorm(D, dtype=dtype, device=device) if qk_norm else None

    def forward(self, x, cos=None, sin=None, positions=None, segment_ids=None, cache=None, layer=None):
        B, S, _ = x.shape
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = self.qkv_proj(x).view(B, S, H + 2 * Hkv, D)
        q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        log_f = F.logsigmoid(self.gate_proj(x).float())                 # [B, S, H]; positions carry no rotation: the gates order the keys
        mask = _causal_mask(S, S, x.device)[None, None]
        if segment_ids is not None:
            mask = mask & (segment_ids[:, :, None] == segment_ids[:, None, :])[:, None]
        out = biased_attention(q, k, v, bias=forgetting_bias(log_f), mask=mask)
        return self.o_proj(out.reshape(B, S, H * D))


# ------------------------------------------------------------------------------------------------ block-selected attention
def moba_selection(q: torch.Tensor, k: torch.Tensor, block: int, top_k: int) -> torch.Tensor:
    """``[B, Hkv, S, top_k]`` key-block indices per query (-1 in a slot that selects none): the query's own block always, then the
    earlier blocks whose mean key scores highest against the query (summed over the group's query heads)."""
    B, S, H, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    nb = (T + block - 1) // block
    pad = nb * block - T
    kb = F.pad(k.float(), (0, 0, 0, 0, 0, pad)).reshape(B, nb, block, Hkv, D)
    count = torch.full((nb,), float(block), device=k.device)
    count[-1] = block - pad
    mean = kb.sum(2) / count[None, :, None, None]                       # [B, nb, Hkv, D]
    g = H // Hkv
    score = torch.einsum("bsgrd,bngd->bgsn", q.float().reshape(B, S, Hkv, g, D), mean)
    own = (torch.arange(S, device=q.device) + (T - S)) // block           # each query's own block
    blocks = torch.arange(nb, device=q.device)
    earlier = blocks[None, :] < own[:, None]                              # strictly before its own (fully visible blocks)
    score = score.masked_fill(~earlier[None, None], float("-inf"))
    k_sel = min(max(top_k - 1, 0), nb)
    if k_sel:
        vals, idx = score.topk(k_sel, -1)
        idx = torch.where(torch.isfinite(vals), idx, torch.full_like(idx, -1))
    else:
        idx = torch.empty(B, Hkv, S, 0, dtype=torch.long, device=q.device)
    return torch.cat([own[None, None, :, None].expand(B, Hkv, S, 1), idx], -1)


def block_sparse_attention(q, k, v, selection: torch.Tensor, block: int, causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """Attention of each query over the keys of its selected blocks (``selection [B, Hkv, S, K]``, -1 = none), causal inside."""
    B, S, H, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    nb = (T + block - 1) // block
    chosen = torch.zeros(B, Hkv, S, nb + 1, dtype=torch.bool, device=q.device)
    chosen.scatter_(3, torch.where(selection >= 0, selection, torch.full_like(selection, nb)), True)
    visible = chosen[..., :nb].repeat_interleave(block, -1)[..., :T]       # [B, Hkv, S, T]
    if causal:
        visible = visible & _causal_mask(S, T, q.device)[None, None]
    mask = visible.repeat_interleave(H // Hkv, 1)
    return biased_attention(q, k, v, mask=mask, scale=scale)


# ------------------------------------------------------------------------------------------------ indexed sparse attention
class LightningIndexer(nn.Module):
    """Scores every key for every query with a few small heads: ``I[t, s] = sum_h w[t, h] relu(q[t, h] . k[s])``."""

    def __init__(self, features: int, heads: int = 4, head_dim: int = 32, dtype=None, device=None):
        super().__init__()
        self.heads, self.head_dim = heads, head_dim
        self.q_proj = Linear(features, heads * head_dim, dtype=dtype, device=device)
        self.k_proj = Linear(features, head_dim, dtype=dtype, device=device)
        self.w_proj = Linear(features, heads, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, _ = x.shape
        q = self.q_proj(x).view(B, S, self.heads, self.head_dim).float()
        k = self.k_proj(x).float()
        w = self.w_proj(x).float() * (self.heads ** -0.5)
        return torch.einsum("bth,bths->bts", w, F.relu(torch.einsum("bthd,bsd->bths", q, k)) * (self.head_dim ** -0.5))


def top_k_selection(scores: torch.Tensor, top_k: int, causal: bool = True) -> torch.Tensor:
    """``scores [B, S, T]`` -> ``[B, S, K]`` key indices per query (-1 where fewer than ``K`` keys are visible)."""
    B, S, T = scores.shape
    if causal:
        scores = scores.masked_fill(~_causal_mask(S, T, scores.device)[None], float("-inf"))
    vals, idx = scores.topk(min(top_k, T), -1)
    return torch.where(torch.isfinite(vals), idx, torch.full_like(idx, -1))


def indexed_sparse_attention(q, k, v, selection: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Attention of each query over its selected keys (``selection [B, S, K]``, -1 = none), shared by every head."""
    B, S, H, D = q.shape
    T = k.shape[1]
    chosen = torch.zeros(B, S, T + 1, dtype=torch.bool, device=q.device)
    chosen.scatter_(2, torch.where(selection >= 0, selection, torch.full_like(selection, T)), True)
    return biased_attention(q, k, v, mask=chosen[:, None, :, :T], scale=scale)


def indexer_alignment_loss(index_scores: torch.Tensor, attention_probs: torch.Tensor, selection: Optional[torch.Tensor] = None) -> torch.Tensor:
    """KL(target || softmax(index scores)) where the target is the main attention's probabilities summed over heads and
    normalised (the indexer's warm-up objective); with ``selection`` both are restricted to the selected keys."""
    B, S, T = index_scores.shape
    target = attention_probs.detach().float().sum(1)
    visible = _causal_mask(S, T, index_scores.device)[None].expand(B, S, T)
    if selection is not None:
        chosen = torch.zeros(B, S, T + 1, dtype=torch.bool, device=index_scores.device)
        chosen.scatter_(2, torch.where(selection >= 0, selection, torch.full_like(selection, T)), True)
        visible = visible & chosen[..., :T]
    target = target * visible
    target = target / target.sum(-1, keepdim=True).clamp_min(1e-12)
    logp = torch.log_softmax(index_scores.float().masked_fill(~visible, float("-inf")), -1)
    logp = torch.where(visible, logp, torch.zeros_like(logp))
    return (target * (target.clamp_min(1e-12).log() - logp)).sum(-1).mean()


# ------------------------------------------------------------------------------------------------ routed value experts
class ValueExperts(nn.Module):
    """The value projection as a mixture: ``v = sum_{e in top_k(router(x))} w_e silu(x W_e)``, the router's selection biased by a
    balance bias that does not enter the weights."""

    def __init__(self, features: int, out_features: int, experts: int = 4, top_k: int = 2, dtype=None, device=None):
        super().__init__()
        self.experts, self.top_k, self.out_features = experts, top_k, out_features
        self.router = Linear(features, experts, dtype=dtype, device=device)
        self.register_buffer("balance_bias", torch.zeros(experts))
        self.weight = nn.Parameter(torch.randn(experts, out_features, features, dtype=dtype, device=device) * features ** -0.5)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        scores = torch.sigmoid(self.router(x).float())
        _, idx = (scores + self.balance_bias).topk(self.top_k, -1)
        w = scores.gather(-1, idx)
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-9)
        dense = torch.zeros_like(scores).scatter(-1, idx, w)                  # [..., E]
        per_expert = F.silu(torch.einsum("...f,eof->...eo", x.float(), self.weight.float()))
        return (dense[..., None] * per_expert).sum(-2).to(x.dtype)
