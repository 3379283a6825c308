"""Decision heads: a score per option, read off a backbone's final states.

Every head takes the backbone's ``[B, L, D]`` final states and the laid-out ``DecisionInputs`` and returns ``[B, Q, K]`` fp32
option logits, unmasked: the caller drops the slots past each question's options.

``DecisionHead``     the question type's embedding is added to the row's states, a few pre-norm transformer blocks (no position
                     encoding, attention inside a row only) run over the window, and each option is scored at its marker
``JointSchemaHead``  decides a row's questions together: options are pooled over their spans and attend to the row (routing
                     layers); each question becomes a field from its instructions, a summary of its options, the row's last
                     token and its type; the fields attend to each other and to the row; option k of question q scores as the
                     scaled product of its routed vector and the field
``LabelReadout``     the backbone's own next-token logits of each option's letter at the answer cue (no new parameters)
``SlotReadout``      ``<slot_k, h> + <q(h), k(m_k)> / sqrt(head_dim)`` with ``h`` the state at the answer cue and ``m_k`` the
                     mean state over option k's span; the slot rows start from the output table's rows of the letters

Reference: src/dew/decision/head.py (``DecisionHead``, ``JointSchemaHead``, ``LabelReadout``, ``SlotReadout``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .inputs import DecisionInputs


def _same_row(seg_q: torch.Tensor, seg_k: torch.Tensor) -> torch.Tensor:
    """[B, Nq, Nk] mask: the query and the key are real and in one row."""
    return (seg_q[:, :, None] == seg_k[:, None, :]) & (seg_k[:, None, :] > 0)


def _attend(q, k, v, heads: int, mask: torch.Tensor) -> torch.Tensor:
    B, Nq, D = q.shape
    hd = D // heads
    qh, kh, vh = (t.reshape(B, t.shape[1], heads, hd).transpose(1, 2) for t in (q, k, v))
    # a query with no key at all (padding) attends to everything rather than producing NaN; its output is never read
    m = mask | ~mask.any(-1, keepdim=True)
    o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=m[:, None])
    return o.transpose(1, 2).reshape(B, Nq, D)


class _Block(nn.Module):
    """Pre-norm block: (self- or cross-) attention, then a feed-forward four times as wide."""

    def __init__(self, d: int, heads: int, cross: bool = False, activation: str = "relu", dropout: float = 0.0):
        super().__init__()
        self.heads, self.cross = heads, cross
        self.norm1, self.norm2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.q, self.kv, self.o = nn.Linear(d, d), nn.Linear(d, 2 * d), nn.Linear(d, d)
        if cross:
            self.norm_c = nn.LayerNorm(d)
            self.cq, self.ckv, self.co = nn.Linear(d, d), nn.Linear(d, 2 * d), nn.Linear(d, d)
        self.up, self.down = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)
        self.act = F.relu if activation == "relu" else F.gelu
        self.drop = nn.Dropout(dropout)

    def forward(self, x, self_mask: Optional[torch.Tensor], memory=None, memory_mask=None):
        if self_mask is not None:
            n = self.norm1(x)
            k, v = self.kv(n).chunk(2, -1)
            x = x + self.drop(self.o(_attend(self.q(n), k, v, self.heads, self_mask)))
        if self.cross:
            n = self.norm_c(x)
            k, v = self.ckv(memory).chunk(2, -1)
            x = x + self.drop(self.co(_attend(self.cq(n), k, v, self.heads, memory_mask)))
        return x + self.drop(self.down(self.act(self.up(self.norm2(x)))))


def _gather(states: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``states [B, L, D]`` at ``index [B, ...]`` -> ``[B, ..., D]``."""
    B, L, D = states.shape
    flat = index.reshape(B, -1).clamp(0, L - 1)
    return states.gather(1, flat[..., None].expand(-1, -1, D)).reshape(*index.shape, D)


def span_means(states: torch.Tensor, start: torch.Tensor, end: torch.Tensor) -> torch.Tensor:
    """Mean of ``states`` over ``[start, end)`` per slot, by a prefix sum (zero for an empty span)."""
    c = torch.cat([torch.zeros_like(states[:, :1]), states.float().cumsum(1)], 1)          # [B, L + 1, D]
    total = _gather(c, end) - _gather(c, start)
    return total / (end - start).clamp_min(1)[..., None]


class Head(nn.Module):
    reads_table = False

    def record(self):
        return {"head": type(self).__name__, **{k: v for k, v in getattr(self, "_fields", {}).items()}}


class DecisionHead(Head):
    def __init__(self, features: int, layers: int = 2, dropout: float = 0.0):
        super().__init__()
        self._fields = {"layers": layers}
        heads = max(1, features // 64)
        self.type_embedding = nn.Embedding(3, features)
        self.blocks = nn.ModuleList([_Block(features, heads, dropout=dropout) for _ in range(layers)])
        self.norm = nn.LayerNorm(features)
        self.score = nn.Linear(features, 1)

    def forward(self, states: torch.Tensor, inputs: DecisionInputs, table=None) -> torch.Tensor:
        x = states.float()
        tk = inputs.token_kind
        x = x + self.type_embedding(tk.clamp_min(0)) * (tk >= 0)[..., None]
        mask = _same_row(inputs.segment_ids, inputs.segment_ids)
        for b in self.blocks:
            x = b(x, mask)
        at = _gather(self.norm(x), inputs.markers)                      # [B, Q, K, D]
        return self.score(at).squeeze(-1).float()


class JointSchemaHead(Head):
    def __init__(self, features: int, width: Optional[int] = None, layers: int = 2, routing_layers: int = 1, dropout: float = 0.0):
        super().__init__()
        d = width or features
        self._fields = {"layers": layers, "routing_layers": routing_layers, "width": d}
        heads = max(1, d // 64)
        self.inp = nn.Linear(features, d)
        self.type_embedding = nn.Embedding(3, d)
        self.routing = nn.ModuleList([_Block(d, heads, cross=True, activation="gelu", dropout=dropout) for _ in range(routing_layers)])
        self.summary = nn.Linear(d, 1)
        self.field = nn.Linear(3 * d, d)
        self.fields = nn.ModuleList([_Block(d, heads, cross=True, activation="gelu", dropout=dropout) for _ in range(layers)])
        self.opt_norm, self.field_norm = nn.LayerNorm(d), nn.LayerNorm(d)
        self.opt_proj, self.field_proj = nn.Linear(d, d, bias=False), nn.Linear(d, d, bias=False)
        self.bias = nn.Linear(d, 1)

    def forward(self, states, inputs: DecisionInputs, table=None):
        B, Q, K = inputs.options.shape
        mem = self.inp(states.float())                                   # [B, L, d]
        d = mem.shape[-1]
        seg = inputs.segment_ids
        opt = span_means(mem, inputs.span_start, inputs.span_end).reshape(B, Q * K, d)
        opt_seg = (inputs.segment_of[:, :, None] * inputs.options).reshape(B, Q * K)
        to_memory = _same_row(opt_seg, seg)
        for layer in self.routing:
            opt = layer(opt, None, mem, to_memory)
        opt = opt.reshape(B, Q, K, d)
        # each question's field: its instructions, an attention-weighted summary of its options, its row's last token, its type
        asked = span_means(mem, inputs.asked_start, inputs.asked_end)
        w = self.summary(opt).squeeze(-1).masked_fill(~inputs.options, float("-inf"))
        w = torch.softmax(torch.where(inputs.options.any(-1, keepdim=True), w, torch.zeros_like(w)), -1) * inputs.options
        summary = (w[..., None] * opt).sum(2)
        last = _gather(mem, inputs.row_end)
        f = self.field(torch.cat([asked, summary, last], -1)) + self.type_embedding(inputs.kinds.clamp_min(0))
        q_seg = inputs.segment_of * (inputs.kinds >= 0)
        among = _same_row(q_seg, q_seg)
        to_mem = _same_row(q_seg, seg)
        for layer in self.fields:
            f = layer(f, among, mem, to_mem)
        o = self.opt_proj(self.opt_norm(opt))
        fq = self.field_proj(self.field_norm(f))
        return ((o * fq[:, :, None]).sum(-1) / math.sqrt(d) + self.bias(self.opt_norm(opt)).squeeze(-1)).float()


class LabelReadout(Head):
    """No parameters: untrained, it is the backbone's own answer.  ``scale`` / ``softcap`` mirror the output table's."""
    reads_table = True

    def __init__(self, softcap: float = 0.0):
        super().__init__()
        self._fields = {"softcap": softcap}
        self.softcap = softcap

    def forward(self, states, inputs: DecisionInputs, table: torch.Tensor = None):
        if inputs.label_ids is None:
            raise ValueError("a label readout needs a lettered layout (Layout(labels=True))")
        if table is None:
            raise ValueError("a label readout reads the backbone's output table")
        h = _gather(states, inputs.readout).float()                      # [B, Q, D]
        rows = table.float()[inputs.label_ids]                          # [B, Q, K, D]
        out = torch.einsum("bqd,bqkd->bqk", h, rows)
        if self.softcap > 0:
            out = self.softcap * torch.tanh(out / self.softcap)
        return out


class SlotReadout(Head):
    reads_table = True

    def __init__(self, features: int, slots: int = 26, head_dim: int = 64):
        super().__init__()
        self._fields = {"slots": slots, "head_dim": head_dim}
        self.slots = nn.Parameter(torch.zeros(slots, features))
        self.q = nn.Linear(features, head_dim, bias=False)
        self.k = nn.Linear(features, head_dim, bias=False)
        nn.init.normal_(self.q.weight, std=features ** -0.5)
        nn.init.normal_(self.k.weight, std=features ** -0.5)
        self.head_dim = head_dim
        self._seeded = False

    def seed_from(self, table: torch.Tensor, label_ids) -> None:
        """Start the slot rows from the output table's rows of the letters."""
        with torch.no_grad():
            ids = torch.as_tensor(label_ids)[: self.slots.shape[0]]
            self.slots[: len(ids)].copy_(table[ids].to(self.slots.dtype))
        self._seeded = True

    def forward(self, states, inputs: DecisionInputs, table=None):
        B, Q, K = inputs.options.shape
        if K > self.slots.shape[0]:
            raise ValueError(f"a question of {K} options is past this readout's {self.slots.shape[0]} slots")
        h = _gather(states, inputs.readout).float()
        m = span_means(states, inputs.span_start, inputs.span_end)      # [B, Q, K, D]
        lex = h @ self.slots[:K].float().t()
        sem = torch.einsum("bqe,bqke->bqk", self.q(h), self.k(m)) / math.sqrt(self.head_dim)
        return lex + sem
