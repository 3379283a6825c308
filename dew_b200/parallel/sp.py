"""Sequence / context parallel attention: positions are split over the ``sequence`` axis; each attention call either
exchanges heads for positions (Ulysses: two all-to-alls) or gathers keys and values with striped causal queries.

Parity: src/dew/nn/attention_parallel.py (``sequence_parallel_attention`` :59-86 chooser, ``all_to_all_moves_less``
:89-116 byte count, ``exchanged_heads_attention`` :223-295, ``gathered_keys_attention`` + ``stripe / unstripe``
:25,298-381).  Ring attention is not offered: the reference measured it 1.04-1.79x slower than all-to-all and rejected
it (docs/guides/multi-node.md:214-223).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops


class _SeqToHeads(torch.autograd.Function):
    """[B, S/N, H, D] -> [B, S, H/N, D] (forward) and back (backward) by one all-to-all."""

    @staticmethod
    def forward(ctx, x, group, to_heads: bool):
        ctx.group, ctx.to_heads = group, to_heads
        return _exchange(x, group, to_heads)

    @staticmethod
    def backward(ctx, g):
        return _exchange(g.contiguous(), ctx.group, not ctx.to_heads), None, None


def _exchange(x, group, to_heads: bool):
    N = dist.get_world_size(group)
    B, S, H, D = x.shape
    if to_heads:      # split heads, gather sequence
        send = x.reshape(B, S, N, H // N, D).permute(2, 0, 1, 3, 4).contiguous()          # [N, B, S, H/N, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.permute(1, 0, 2, 3, 4).reshape(B, N * S, H // N, D)                    # rank-major positions
    send = x.reshape(B, N, S // N, H, D).permute(1, 0, 2, 3, 4).contiguous()               # [N, B, S/N, H, D]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 2, 0, 3, 4).reshape(B, S // N, N * H, D)


def exchanged_heads_attention(q, k, v, group=None, causal: bool = True, **kw):
    """Ulysses: all-to-all positions<->heads, full-sequence attention on ``H / N`` heads, all-to-all back."""
    N = dist.get_world_size(group)
    if q.shape[2] % N or k.shape[2] % N:
        raise ValueError(f"heads {q.shape[2]} / {k.shape[2]} do not divide by the sequence-parallel size {N}")
    qh, kh, vh = (_SeqToHeads.apply(t, group, True) for t in (q, k, v))
    o = ops.attention(qh, kh, vh, causal=causal, **kw)
    return _SeqToHeads.apply(o, group, False)


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, 1)

    @staticmethod
    def backward(ctx, g):
        N, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        S = g.shape[1] // N
        return g[:, r * S:(r + 1) * S], None


def stripe(x: torch.Tensor, N: int) -> torch.Tensor:
    """Reorder positions so that rank ``r`` holds chunks ``r`` and ``2N - 1 - r`` of ``2N``: balanced causal work."""
    B, S = x.shape[:2]
    c = x.reshape(B, 2 * N, S // (2 * N), *x.shape[2:])
    order = [i for r in range(N) for i in (r, 2 * N - 1 - r)]
    return c[:, order].reshape(x.shape)


def unstripe(x: torch.Tensor, N: int) -> torch.Tensor:
    B, S = x.shape[:2]
    c = x.reshape(B, 2 * N, S // (2 * N), *x.shape[2:])
    order = [i for r in range(N) for i in (r, 2 * N - 1 - r)]
    inv = [order.index(i) for i in range(2 * N)]
    return c[:, inv].reshape(x.shape)


def gathered_keys_attention(q, k, v, positions, group=None, causal: bool = True):
    """Keys / values are all-gathered; every rank attends its own (striped) queries to the whole sequence using the
    absolute ``positions [B, S_local]`` of its queries for the causal mask."""
    kf, vf = _GatherSeq.apply(k, group), _GatherSeq.apply(v, group)
    N = dist.get_world_size(group)
    pos_parts = [torch.empty_like(positions) for _ in range(N)]
    dist.all_gather(pos_parts, positions.contiguous(), group=group)
    kpos = torch.cat(pos_parts, 1)                                             # [B, S] absolute position of each key
    B, S, Hq, D = q.shape
    rep = Hq // kf.shape[2]
    s = torch.einsum("bshd,bthd->bhst", q.float(), kf.float().repeat_interleave(rep, 2)) / (D ** 0.5)
    if causal:
        mask = kpos[:, None, None, :] <= positions[:, None, :, None]
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    return torch.einsum("bhst,bthd->bshd", p, vf.float().repeat_interleave(rep, 2)).to(q.dtype)


def all_to_all_moves_less(seq: int, heads: int, kv_heads: int, head_dim: int, N: int) -> bool:
    """Byte count of the two schemes per rank: Ulysses moves q, k, v, o once; gathered-keys moves k, v (N - 1) times."""
    ulysses = (2 * heads + 2 * kv_heads) * seq // N * head_dim * (N - 1) / N
    gathered = 2 * kv_heads * seq // N * head_dim * (N - 1)
    return ulysses <= gathered


def sequence_parallel_attention(q, k, v, positions=None, group=None, causal: bool = True):
    """Pick the exchange: Ulysses when the heads divide and it moves fewer bytes, else gathered keys."""
    N = dist.get_world_size(group) if dist.is_initialized() else 1
    if N == 1:
        return ops.attention(q, k, v, causal=causal)
    heads_ok = q.shape[2] % N == 0 and k.shape[2] % N == 0
    if heads_ok and (positions is None or all_to_all_moves_less(q.shape[1] * N, q.shape[2], k.shape[2], q.shape[3], N)):
        return exchanged_heads_attention(q, k, v, group, causal)
    if positions is None:
        r = dist.get_rank(group)
        positions = (torch.arange(q.shape[1], device=q.device) + r * q.shape[1])[None].expand(q.shape[0], -1)
    return gathered_keys_attention(q, k, v, positions, group, causal)
