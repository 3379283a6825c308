"""Sequence-parallel pieces beyond attention, and two vocabulary / feature-parallel reductions.  Positions are split in
contiguous blocks over the ranks of a group (rank r holds positions ``[r S / N, (r + 1) S / N)``).

``sequence_halo``                 the last ``width`` positions of the previous rank (zeros on rank 0), differentiable
``sequence_parallel_short_conv``  causal depthwise convolution whose taps reach into the previous rank's block
``banded_attention``              sliding-window attention whose window reaches into the previous rank's block
``sequence_parallel_scan``        a linear recurrence across ranks: every rank runs its block from the state the previous
                                  rank hands over (gated delta rule, SSD: any ``fn(initial_state) -> (out, final_state)``);
                                  the hand-off is a differentiable send / receive, so the backward walks the ranks in reverse
``vocab_parallel_cross_entropy``  the head's vocabulary split over ranks: max, sum of exponentials and the target logit are
                                  reduced, the full logits never exist on one rank
``sharded_rms_norm``              RMSNorm over a feature axis split over ranks (sum of squares reduced)

Reference: src/dew/nn/linear.py:696-781 (``sequence_halo`` :734, ``sequence_delta_rule`` :781), src/dew/nn/local_attention.py:307
(halo exchange), src/dew/nn/kernels/recurrence_algebra.py:367-370 (state scan across the sequence axis),
src/dew/objectives/lm/chunked.py:411-429,1143-1228 (vocabulary split), src/dew/nn/norms.py:429 (sharded statistics).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops
from ..ops import scan

_LINK = None


def use_peer_link(link) -> None:
    """Route this module's exchanges through a ``parallel.peer_link.PeerLink`` (one kernel per exchange over NVLink peer memory,
    arrival tags inside the data) instead of ``torch.distributed`` point-to-point calls; ``None`` switches back.  The link's group
    must be the group the functions are called with."""
    global _LINK
    _LINK = link


def _linked(x: torch.Tensor, group) -> bool:
    return _LINK is not None and _LINK.group is group and x.is_cuda


class _ShiftFromPrevious(torch.autograd.Function):
    """out on rank r = x of rank r - 1 (zeros on rank 0); backward shifts the gradient the other way."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _shift(x.contiguous(), group, +1)

    @staticmethod
    def backward(ctx, g):
        return _shift(g.contiguous(), ctx.group, -1), None


def _shift(x: torch.Tensor, group, direction: int) -> torch.Tensor:
    """direction +1: receive from rank - 1, send to rank + 1; -1: the reverse.  Edge ranks receive zeros."""
    rank, N = dist.get_rank(group), dist.get_world_size(group)
    src, dst = rank - direction, rank + direction
    if _linked(x, group):
        got = _LINK.exchange(x, dst if 0 <= dst < N else None, src if 0 <= src < N else None)
        return got if got is not None else torch.zeros_like(x)
    out = torch.zeros_like(x)
    ops_ = []
    if 0 <= dst < N:
        ops_.append(dist.P2POp(dist.isend, x, dist.get_global_rank(group, dst) if group is not None else dst, group))
    if 0 <= src < N:
        ops_.append(dist.P2POp(dist.irecv, out, dist.get_global_rank(group, src) if group is not None else src, group))
    if ops_:
        for w in dist.batch_isend_irecv(ops_):
            w.wait()
    return out


def sequence_halo(x: torch.Tensor, width: int, group=None) -> torch.Tensor:
    """``x [B, S_local, ...]`` -> the previous rank's last ``width`` positions ``[B, width, ...]`` (zeros on rank 0)."""
    return _ShiftFromPrevious.apply(x[:, -width:], group)


def sequence_parallel_short_conv(x, w, bias=None, activation: bool = True, group=None):
    """Causal depthwise conv over a sequence split across ranks: ``x [B, S_local, C]``, ``w [C, K]``."""
    K = w.shape[1]
    halo = sequence_halo(x, K - 1, group)
    # rank 0's halo is zeros, which is the causal left padding; every rank takes the same path so that every rank's backward
    # runs the matching shift
    y = scan.short_conv(torch.cat([halo, x], 1), w, bias, activation)
    return y[:, K - 1:]


def banded_attention(q, k, v, window: int, group=None, scale: Optional[float] = None):
    """Causal sliding-window attention (each query sees its last ``window`` keys) with the sequence split across ranks; the
    window may not exceed a rank's block, so one halo from the previous rank suffices."""
    S = q.shape[1]
    if window > S:
        raise ValueError(f"window {window} exceeds the local block of {S} positions: it would reach past the previous rank")
    kh, vh = sequence_halo(k, window, group), sequence_halo(v, window, group)
    kk, vv = torch.cat([kh, k], 1), torch.cat([vh, v], 1)
    # query i (local) sits at position window + i of the extended keys; on rank 0 the halo is zeros and must be masked
    T = kk.shape[1]
    qi = torch.arange(S, device=q.device)[:, None] + window
    kj = torch.arange(T, device=q.device)[None, :]
    mask = (kj <= qi) & (kj > qi - window)
    if dist.get_rank(group) == 0:
        mask = mask & (kj >= window)
    Hq, Hkv = q.shape[2], k.shape[2]
    kk, vv = (t.repeat_interleave(Hq // Hkv, 2) for t in (kk, vv))
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    s = torch.einsum("bihd,bjhd->bhij", q.float(), kk.float()) * scale
    s = s.masked_fill(~mask[None, None], float("-inf"))
    return torch.einsum("bhij,bjhd->bihd", torch.softmax(s, -1), vv.float()).to(q.dtype)


class _HandOver(torch.autograd.Function):
    """Receive the state from rank - 1 (forward) and send its gradient back to rank - 1 (backward).  The argument only
    carries shape, dtype and the autograd edge."""

    @staticmethod
    def forward(ctx, like, group):
        ctx.group = group
        rank = dist.get_rank(group)
        src = rank - 1
        if _linked(like, group):
            return _LINK.exchange(None, None, src, like=like.detach())
        buf = torch.zeros_like(like)
        dist.recv(buf, dist.get_global_rank(group, src) if group is not None else src, group=group)
        return buf

    @staticmethod
    def backward(ctx, g):
        rank = dist.get_rank(ctx.group)
        dst = rank - 1
        if _linked(g, ctx.group):
            _LINK.exchange(g.contiguous(), dst, None)
            return torch.zeros_like(g), None
        dist.send(g.contiguous(), dist.get_global_rank(ctx.group, dst) if ctx.group is not None else dst, group=ctx.group)
        return torch.zeros_like(g), None


def sequence_parallel_scan(fn: Callable[[Optional[torch.Tensor]], Tuple[torch.Tensor, torch.Tensor]], state_like: torch.Tensor, group=None):
    """Run ``fn(initial_state) -> (out, final_state)`` on every rank in rank order, each starting from its predecessor's final
    state (rank 0 starts from ``None``).  ``state_like`` gives the state's shape / dtype / device.  A rank's receive blocks until
    its predecessor has finished (the recurrence is sequential across the sequence); in the backward the gradient of the
    state travels the other way."""
    rank, N = dist.get_rank(group), dist.get_world_size(group)
    incoming = None
    if rank > 0:
        # receive the predecessor's final state: the matching send is the predecessor's _HandOver below
        incoming = _HandOver.apply(torch.zeros_like(state_like).requires_grad_(state_like.is_floating_point()), group)
    out, final = fn(incoming)
    if rank < N - 1:
        # hand the state to the successor; the result (what the predecessor sent) is already consumed above, so it is dropped
        sent = _HandOverSend.apply(final, group)
        out = out + 0 * sent.sum().to(out.dtype)         # keeps the send in the autograd graph so that its backward runs
    return out, final


class _HandOverSend(torch.autograd.Function):
    """Send ``x`` to rank + 1 (forward) and receive the gradient of it from rank + 1 (backward)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group, ctx.shape, ctx.dtype = group, x.shape, x.dtype
        rank = dist.get_rank(group)
        dst = rank + 1
        if _linked(x, group):
            _LINK.exchange(x.contiguous(), dst, None)
            return x.new_zeros(())
        dist.send(x.contiguous(), dist.get_global_rank(group, dst) if group is not None else dst, group=group)
        return x.new_zeros(())

    @staticmethod
    def backward(ctx, g):
        rank = dist.get_rank(ctx.group)
        src = rank + 1
        if _linked(g, ctx.group):
            return _LINK.exchange(None, None, src, like=torch.empty(ctx.shape, dtype=ctx.dtype, device=g.device)), None
        buf = torch.zeros(ctx.shape, dtype=g.dtype, device=g.device)
        dist.recv(buf, dist.get_global_rank(ctx.group, src) if ctx.group is not None else src, group=ctx.group)
        return buf, None


def vocab_parallel_cross_entropy(hidden: torch.Tensor, weight_shard: torch.Tensor, targets: torch.Tensor, group=None,
                                 ignore_index: int = -100) -> Tuple[torch.Tensor, torch.Tensor]:
    """``hidden [T, d]``, ``weight_shard [V / N, d]`` (rank r holds vocabulary rows ``[r V / N, (r + 1) V / N)``), ``targets [T]``
    (global ids) -> (summed loss, number of scored targets); differentiable w.r.t. hidden and the shard."""
    rank, N = dist.get_rank(group), dist.get_world_size(group)
    Vs = weight_shard.shape[0]
    logits = hidden.float() @ weight_shard.float().t()                          # [T, V / N]
    local_max = logits.max(-1).values.detach()
    if _linked(local_max, group):
        gmax = _LINK.all_reduce(local_max, "max")
    else:
        gmax = local_max.clone()
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
    sumexp = _AllReduceSum.apply(torch.exp(logits - gmax[:, None]).sum(-1), group)
    lo = rank * Vs
    mine = (targets >= lo) & (targets < lo + Vs)
    picked = logits.gather(-1, (targets - lo).clamp(0, Vs - 1)[:, None])[:, 0]
    target_logit = _AllReduceSum.apply(torch.where(mine, picked, torch.zeros_like(picked)), group)
    scored = targets != ignore_index
    nll = torch.log(sumexp) + gmax - target_logit
    return torch.where(scored, nll, torch.zeros_like(nll)).sum(), scored.sum()


class _AllReduceSum(torch.autograd.Function):
    """Sum over ranks whose backward passes the gradient through unchanged (every rank holds the same result)."""

    @staticmethod
    def forward(ctx, x, group):
        if _linked(x, group) and x.dtype == torch.float32:
            return _LINK.all_reduce(x, "sum")
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def sharded_rms_norm(x_shard: torch.Tensor, w_shard: torch.Tensor, features: int, eps: float = 1e-6, group=None) -> torch.Tensor:
    """RMSNorm over a feature axis of total width ``features`` of which this rank holds ``x_shard [..., features / N]``."""
    ss = _AllReduceSum.apply(x_shard.float().pow(2).sum(-1, keepdim=True), group)
    return (x_shard.float() * torch.rsqrt(ss / features + eps) * w_shard.float()).to(x_shard.dtype)
