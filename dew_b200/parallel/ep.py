"""Expert parallelism: the experts of every sparse layer are split over the ``expert`` axis; tokens travel to the rank
that owns their expert and back.

Protocol (what ``ExpertParallel.dispatch_compute_combine`` does):
  1. every rank counts its (token, choice) pairs per expert and all ranks exchange the ``[W, E]`` count matrix (tiny);
     from it every rank derives the same placement: on the owner of expert ``e`` the rows arriving from rank ``r`` sit at
     ``aligned_offset[e] + sum_{r' < r} counts[r'][e]`` of an expert-sorted, 128-aligned buffer - so arriving rows land
     *directly* in the layout the tcgen05 grouped GEMM consumes;
  2. dispatch: rows are sent (all-to-all with uneven splits; on GPUs the peer-memory push kernel writes them straight
     into the destination's buffer);
  3. the owner runs the grouped gate|up GEMM, SwiGLU, grouped down GEMM on its local experts;
  4. combine: the result rows return to their source ranks and are summed per token with the routing weights.
Everything is differentiable (the backward of a dispatch is a combine and vice versa).

Reference behaviour: ``dispatch='exchange'`` with ``ragged_all_to_all`` rounds (src/dew/nn/moe.py:1131-1215), per-expert
count all-gather (:1168), capacity factor (docs/concepts/moe.md:95).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import grouped as G


class _AllToAll(torch.autograd.Function):
    """Uneven all-to-all of rows; the backward is the all-to-all with the split lists swapped."""

    @staticmethod
    def forward(ctx, x, send_splits: List[int], recv_splits: List[int], group):
        ctx.send, ctx.recv, ctx.group = send_splits, recv_splits, group
        out = x.new_empty((sum(recv_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv, group=ctx.group)
        return out, None, None, None


def all_to_all_rows(x, send_splits, recv_splits, group=None):
    return _AllToAll.apply(x, list(send_splits), list(recv_splits), group)


class ExpertParallel:
    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    # ------------------------------------------------------------------ sharding the experts of a model
    def shard(self, model) -> None:
        """Keep only this rank's slice of every ``ExpertMLP`` (experts ``[rank * E / W, (rank + 1) * E / W)``)."""
        from ..nn.moe import SparseMLP
        for m in model.modules():
            if isinstance(m, SparseMLP):
                E = m.mix.experts
                if E % self.world:
                    raise ValueError(f"{E} experts do not divide over {self.world} expert-parallel ranks")
                per = E // self.world
                lo = self.rank * per
                ex = m.experts
                ex.gate_up = torch.nn.Parameter(ex.gate_up.data[lo:lo + per].clone(), requires_grad=ex.gate_up.requires_grad)
                ex.down = torch.nn.Parameter(ex.down.data[lo:lo + per].clone(), requires_grad=ex.down.requires_grad)
                ex.gate_up.expert_parallel = ex.down.expert_parallel = True      # gradients are NOT averaged over this axis
                ex.experts_n = per
                m.ep = self

    # ------------------------------------------------------------------ the exchange
    def dispatch_compute_combine(self, mlp, x2: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        W, E = self.world, mlp.mix.experts
        per = E // W
        T, k = ids.shape
        flat = ids.reshape(-1)
        # sort this rank's pairs by expert: contiguous by destination rank, and by expert within a rank
        order = torch.argsort(flat, stable=True)
        sorted_ids = flat[order]
        rows = x2.index_select(0, order // k)
        counts = torch.bincount(flat, minlength=E)
        if W > 1:
            parts = [torch.empty_like(counts) for _ in range(W)]
            dist.all_gather(parts, counts.contiguous(), group=self.group)
            all_counts = torch.stack(parts, 0)
        else:
            all_counts = counts[None]
        send = counts.reshape(W, per).sum(1).tolist()
        mine = all_counts[:, self.rank * per:(self.rank + 1) * per]            # [W sources, local experts]
        recv = mine.sum(1).tolist()
        got = all_to_all_rows(rows, send, recv, self.group) if W > 1 else rows
        # expert of every received row: sources arrive in rank order, each sorted by expert
        local_ids = torch.cat([torch.repeat_interleave(torch.arange(per, device=ids.device), mine[r]) for r in range(W)]) \
            if got.shape[0] else torch.zeros(0, dtype=torch.long, device=ids.device)
        layout = G.group_layout(local_ids, per)
        buf = torch.zeros((layout.rows, x2.shape[1]), dtype=x2.dtype, device=x2.device).index_copy(0, layout.positions, got)
        out = mlp.experts(buf, layout).index_select(0, layout.positions)
        back = all_to_all_rows(out, recv, send, self.group) if W > 1 else out
        # undo the sort and combine with the routing weights
        unsorted = torch.empty_like(back).index_copy(0, order, back)
        return (unsorted.reshape(T, k, -1).float() * weights.float().unsqueeze(-1)).sum(1).to(x2.dtype)
