"""Grouped (per-expert) GEMMs over token rows sorted by expert, for mixture-of-experts layers.

Layout: tokens routed to expert ``g`` occupy rows ``[offsets[g], offsets[g] + counts[g])`` of a padded buffer whose
group starts are multiples of 128 and whose padding rows are zero, so the tcgen05 kernel's 128-row tiles never
straddle experts and the weight gradient's reduction never reads a neighbour's rows
(capabilities of src/dew/nn/kernels/grouped_matmul.py ``gmm`` / ``tgmm``; kernels/cutlass/ffi.cu:176-256).
Everything here is device-side: no host synchronisation on the routing counts.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


def _grad_accumulates(p) -> bool:
    from .functional import grad_accumulates
    return grad_accumulates(p)

from . import library as L

c_ll, c_int, c_float = ctypes.c_longlong, ctypes.c_int, ctypes.c_float
BLOCK = 128


@dataclass
class GroupLayout:
    """Where every (token, choice) pair sits in the expert-sorted padded buffer."""
    positions: torch.Tensor      # [T * k] int64: padded row of each (token, choice), in (token, choice) order
    counts: torch.Tensor         # [G] int32 rows per expert
    offsets: torch.Tensor        # [G + 1] int32 aligned start of each expert (offsets[G] = rows in use, aligned)
    tile_group: torch.Tensor     # [rows / 128] int32 expert of each 128-row tile, -1 past the rows in use
    rows: int                    # static size of the padded buffer


def padded_rows(pairs: int, groups: int, block: int = BLOCK) -> int:
    """Static upper bound of the padded buffer: every group may waste up to ``block - 1`` rows."""
    return ((pairs + groups * (block - 1)) + block - 1) // block * block


def group_layout(expert_ids: torch.Tensor, groups: int, block: int = BLOCK) -> GroupLayout:
    """``expert_ids [pairs]`` (expert of each (token, choice)) -> aligned expert-sorted layout, all on device."""
    pairs = expert_ids.numel()
    ids = expert_ids.reshape(-1).to(torch.int64)
    counts = torch.bincount(ids, minlength=groups)
    aligned = (counts + block - 1) // block * block
    offsets = torch.zeros(groups + 1, dtype=torch.int64, device=ids.device)
    offsets[1:] = torch.cumsum(aligned, 0)
    order = torch.argsort(ids, stable=True)
    start_unaligned = torch.cumsum(counts, 0) - counts
    rank_in_group = torch.empty_like(order)
    rank_in_group[order] = torch.arange(pairs, device=ids.device) - start_unaligned[ids[order]]
    positions = offsets[ids] + rank_in_group
    rows = padded_rows(pairs, groups, block)
    tiles = rows // block
    tile_start = torch.arange(tiles, device=ids.device, dtype=torch.int64) * block
    tile_group = torch.searchsorted(offsets[1:].contiguous(), tile_start, right=True)
    tile_group = torch.where(tile_start < offsets[-1], tile_group, torch.full_like(tile_group, -1))
    return GroupLayout(positions, counts.to(torch.int32), offsets.to(torch.int32), tile_group.to(torch.int32), rows)


def _gmm_reference(x, w, layout: GroupLayout, transpose_w: bool):
    """fp32 loop over groups (CPU oracle): rows of group g times w[g]^T (or w[g] when ``transpose_w``)."""
    out_features = w.shape[2] if transpose_w else w.shape[1]
    out = torch.zeros((x.shape[0], out_features), dtype=torch.float32, device=x.device)
    off = layout.offsets.tolist()
    cnt = layout.counts.tolist()
    for g in range(w.shape[0]):
        r0, n = off[g], cnt[g]
        if n:
            wg = w[g].float()
            out[r0:r0 + n] = x[r0:r0 + n].float() @ (wg if transpose_w else wg.t())
    return out.to(x.dtype)


def _tgmm_reference(dy, x, layout: GroupLayout, groups: int):
    off = layout.offsets.tolist()
    cnt = layout.counts.tolist()
    out = torch.zeros((groups, dy.shape[1], x.shape[1]), dtype=torch.float32, device=x.device)
    for g in range(groups):
        r0, n = off[g], cnt[g]
        if n:
            out[g] = dy[r0:r0 + n].float().t() @ x[r0:r0 + n].float()
    return out


def gmm_forward(x, w, layout: GroupLayout, transpose_w: bool = False, out=None):
    """``out[rows of g] = x[rows of g] @ w[g]^T`` (``w [G, N, K]``) or ``@ w[g]`` (``w [G, K, N]``, ``transpose_w``)."""
    if not L.use_cuda(x, w):
        return _gmm_reference(x, w, layout, transpose_w)
    G = w.shape[0]
    M, K = x.shape
    N = w.shape[2] if transpose_w else w.shape[1]
    if out is None:
        out = torch.zeros((M, N), dtype=torch.bfloat16, device=x.device)    # tiles past the rows in use are skipped
    w2 = w.reshape(G * w.shape[1], w.shape[2])
    rc = L.load().dewb_gmm_bf16(L.ptr(x), L.ptr(w2), L.ptr(out), L.ptr(layout.tile_group), c_int(M), c_int(N), c_int(K),
                                c_int(G), c_ll(x.stride(0)), c_ll(w2.stride(0)), c_ll(out.stride(0)),
                                c_int(int(transpose_w)), c_int(0), c_float(1.0), L.ptr(L.status(x.device)), L.stream_ptr())
    L.check(rc, "gmm_bf16")
    L.count_launches()
    return out


def tgmm(dy, x, layout: GroupLayout, groups: int, out: Optional[torch.Tensor] = None, accumulate: bool = False):
    """Per-group ``dW[g] = dy[rows of g]^T @ x[rows of g]`` -> ``[G, N, K]`` (fp32 when accumulating into ``out``)."""
    if not L.use_cuda(dy, x):
        r = _tgmm_reference(dy, x, layout, groups)
        if out is not None:
            out.add_(r.to(out.dtype)) if accumulate else out.copy_(r.to(out.dtype))
            return out
        return r.to(dy.dtype)
    R, N = dy.shape
    K = x.shape[1]
    if out is None:
        out = torch.empty((groups, N, K), dtype=torch.bfloat16, device=dy.device)
        accumulate = False
    epi = {(torch.bfloat16, False): 0, (torch.float32, False): 1, (torch.float32, True): 2, (torch.bfloat16, True): 3}[(out.dtype, accumulate)]
    rc = L.load().dewb_tgmm_bf16(L.ptr(dy), L.ptr(x), L.ptr(out), L.ptr(layout.offsets), c_int(R), c_int(N), c_int(K),
                                 c_int(groups), c_ll(dy.stride(0)), c_ll(x.stride(0)), c_ll(out.stride(1)),
                                 c_ll(out.stride(0)), c_int(epi), c_float(1.0), L.ptr(L.status(dy.device)), L.stream_ptr())
    L.check(rc, "tgmm_bf16")
    L.count_launches()
    return out


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, layout):
        ctx.layout = layout
        ctx.save_for_backward(x, w)
        return gmm_forward(x, w, layout)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        layout = ctx.layout
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gmm_forward(dy, w, layout, transpose_w=True)            # dy [M, N] @ w[g] [N, K]
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            if main is not None and dy.is_cuda:
                tgmm(dy, x, layout, w.shape[0], out=main, accumulate=_grad_accumulates(w))
            else:
                dw = tgmm(dy, x, layout, w.shape[0]).to(w.dtype)
        return dx, dw, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, layout: GroupLayout) -> torch.Tensor:
    """Differentiable per-expert linear on an expert-sorted padded buffer: ``x [rows, K]``, ``w [G, N, K]``."""
    return _GroupedLinear.apply(x, w, layout)


def permute(x: torch.Tensor, layout: GroupLayout, top_k: int) -> torch.Tensor:
    """Scatter token rows into the padded expert-sorted buffer (each token appears ``top_k`` times); padding is zero."""
    T, d = x.shape
    buf = torch.zeros((layout.rows, d), dtype=x.dtype, device=x.device)
    src = x.repeat_interleave(top_k, 0) if top_k > 1 else x
    return buf.index_copy(0, layout.positions, src)


def combine(y: torch.Tensor, layout: GroupLayout, weights: torch.Tensor, tokens: int) -> torch.Tensor:
    """``out[t] = sum_k weights[t, k] * y[position(t, k)]`` (fp32 accumulate, result in ``y``'s dtype)."""
    k = weights.shape[1]
    rows = y.index_select(0, layout.positions).reshape(tokens, k, y.shape[1])
    return (rows.float() * weights.float().unsqueeze(-1)).sum(1).to(y.dtype)
