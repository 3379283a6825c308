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

import ctypes
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import grouped as G
from ..ops import library as L
from .symm import SymmetricBuffer


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


class _LocalBuffer:
    """Plain device memory with the interface of ``SymmetricBuffer``, for an exchange that spans one rank."""

    def __init__(self, numel: int, dtype, device):
        self.tensor = torch.zeros(numel, dtype=dtype, device=device)

    def ptr_array(self, offset_bytes: int = 0):
        return (ctypes.c_ulonglong * 8)(*([self.tensor.data_ptr() + offset_bytes] + [0] * 7))


class ExchangePlan:
    """Where every (token, choice) pair goes: destination rank and row, plus this rank's layout as an owner."""

    def __init__(self, dest_rank, dest_pos, layout, info, tokens: int, top_k: int):
        self.dest_rank, self.dest_pos, self.layout, self.info = dest_rank, dest_pos, layout, info
        self.tokens, self.top_k = tokens, top_k


class TokenExchange:
    """Dispatch and combine of expert rows through peer memory, planned on the device (no host synchronisation).

    ``plan``  ranks every pair inside its expert, exchanges the per-expert counts through symmetric memory and derives
              the placement every rank agrees on;
    ``push``  stores token rows straight into the owners' expert-sorted receive buffers (peer stores) and returns this
              rank's received rows;
    ``pull``  loads each token's result rows from the owners' output buffers (peer loads) and sums them with the
              routing weights.
    One rank runs the same kernels with itself as the only peer.  Shapes must be the same on every rank of the group.
    The receive buffer holds ``capacity_factor`` times a rank's fair share of rows (all of them with one rank); pairs
    past its end are dropped and the device status word reports it.
    Kernels: ``csrc/kernels/moe_sm100.cu``."""

    SLOT_COUNTS, SLOT_READY, SLOT_PUSHED, SLOT_OUT, SLOT_PULLED = 0, 1, 2, 3, 4

    def __init__(self, experts: int, group: Optional[dist.ProcessGroup] = None, capacity_factor: float = 2.0, wait_limit_s: float = 20.0):
        local = isinstance(group, str) and group == "self"           # a one-rank exchange inside a larger job
        self.group = None if local else group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and not local) else 1
        self.rank = dist.get_rank(group) if (dist.is_initialized() and not local) else 0
        self.local = local
        if experts % self.world:
            raise ValueError(f"{experts} experts do not divide over {self.world} ranks")
        self.experts, self.per = experts, experts // self.world
        self.capacity_factor = capacity_factor
        self.limit_ns = int(wait_limit_s * 1e9)
        self.seq = 0
        self.last_pull = 0
        self.rows_cap = 0
        self.features = 0
        self.recv = self.recv_back = self.out = self.counts = self.flags = None
        # lean buffers (DEWB_EP_LEAN=0 restores the copies): the receive buffer is returned as it is (a second one takes the
        # backward's rows, so the forward's stay intact for the weight gradient), only the padding rows of each expert group are
        # zeroed instead of the whole buffer, and the last expert product may write straight into the buffer the peers pull from
        self.lean = os.environ.get("DEWB_EP_LEAN", "1") == "1"
        self.write_in_place = os.environ.get("DEWB_EP_IN_PLACE", "1") == "1"      # the last expert product writes into the pulled buffer
        self._out_claimed = False

    def _ensure(self, pairs: int, features: int, device) -> None:
        share = pairs if self.world == 1 else int(pairs * self.capacity_factor)
        need = G.padded_rows(share, self.per)
        if self.recv is not None and need <= self.rows_cap and features == self.features:
            return
        self.rows_cap, self.features = need, features
        make = (lambda n, dt: _LocalBuffer(n, dt, device)) if self.world == 1 else \
            (lambda n, dt: SymmetricBuffer(n, dt, device, self.group, zero=True))
        # (one row more than the plan addresses: the target of the padding-zeroing writes that have nothing to zero)
        self.recv, self.out = make((need + 1) * features, torch.bfloat16), make(need * features, torch.bfloat16)
        self.recv_back = make((need + 1) * features, torch.bfloat16) if self.lean else None
        if self.counts is None:
            self.counts, self.flags = make(max(64, self.experts), torch.int32), make(64, torch.int32)
            self.counter = torch.zeros(4, dtype=torch.int32, device=device)

    def _signal(self, slot: int) -> None:
        if self.world > 1:
            L.check(L.load().dewb_signal_flags(self.flags.ptr_array(), ctypes.c_int(slot), ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                               ctypes.c_uint(self.seq), L.stream_ptr()), "signal_flags")

    def _wait(self, slot: int, seq: int) -> None:
        if self.world > 1:
            L.check(L.load().dewb_wait_flags(L.ptr(self.flags.tensor), ctypes.c_int(slot), ctypes.c_int(self.world), ctypes.c_uint(seq),
                                             ctypes.c_ulonglong(self.limit_ns), L.ptr(L.status(self.flags.tensor.device)), L.stream_ptr()),
                    "wait_flags")

    def plan(self, ids: torch.Tensor, features: int) -> ExchangePlan:
        T, k = ids.shape
        pairs = T * k
        dev = ids.device
        L.ensure_device(ids)
        self._ensure(pairs, features, dev)
        lib = L.load()
        ids32 = ids.to(torch.int32).contiguous().reshape(-1)
        rank_in_group = torch.empty(pairs, dtype=torch.int32, device=dev)
        self.seq += 1
        L.check(lib.dewb_moe_rank(L.ptr(ids32), ctypes.c_int(pairs), ctypes.c_int(self.experts), L.ptr(rank_in_group),
                                  L.ptr(self.counts.tensor), L.stream_ptr()), "moe_rank")
        self._signal(self.SLOT_COUNTS)
        dest_rank = torch.empty(pairs, dtype=torch.int32, device=dev)
        dest_pos = torch.empty(pairs, dtype=torch.int32, device=dev)
        offsets = torch.empty(self.per + 1, dtype=torch.int32, device=dev)
        local_counts = torch.empty(self.per, dtype=torch.int32, device=dev)
        tile_group = torch.empty(self.rows_cap // 128, dtype=torch.int32, device=dev)
        info = torch.zeros(4, dtype=torch.int32, device=dev)     # {rows received, overflowed, busiest owner's rows, pairs dropped}
        L.check(lib.dewb_moe_plan(self.counts.ptr_array(), L.ptr(self.flags.tensor), ctypes.c_int(self.SLOT_COUNTS), ctypes.c_uint(self.seq),
                                  ctypes.c_ulonglong(self.limit_ns), L.ptr(ids32), L.ptr(rank_in_group), ctypes.c_int(pairs),
                                  ctypes.c_int(self.experts), ctypes.c_int(self.rank), ctypes.c_int(self.world), ctypes.c_int(self.rows_cap),
                                  L.ptr(dest_rank), L.ptr(dest_pos), L.ptr(offsets), L.ptr(local_counts), L.ptr(tile_group), L.ptr(info),
                                  L.ptr(L.status(dev)), L.stream_ptr()), "moe_plan")
        L.count_launches(2)
        layout = G.GroupLayout(None, local_counts, offsets, tile_group, self.rows_cap)
        plan = ExchangePlan(dest_rank, dest_pos, layout, info, T, k)
        if self.lean:
            # rows [offset + count, next offset) of every local expert: the (at most 127) alignment rows nobody pushes; a fixed-size
            # index (entries with nothing to zero point at the spare row) keeps this free of data-dependent shapes
            j = torch.arange(127, device=dev, dtype=torch.int64)[None, :]
            first = (offsets[:-1] + local_counts).long()[:, None] + j
            plan.pad_rows = torch.where(first < offsets[1:].long()[:, None], first, self.rows_cap).reshape(-1)
        return plan

    def push(self, x: torch.Tensor, plan: ExchangePlan, pair_scale: Optional[torch.Tensor] = None, backward: bool = False) -> torch.Tensor:
        """``x [T, d]`` bf16 -> this rank's received rows ``[rows_cap, d]`` (expert-sorted, padding rows zero)."""
        T, d = x.shape
        assert d == self.features and x.dtype == torch.bfloat16
        L.ensure_device(x)
        self.seq += 1
        buf = self.recv_back if (self.lean and backward) else self.recv
        if not self.lean:
            buf.tensor.zero_()
        self._signal(self.SLOT_READY)
        ps = None if pair_scale is None else pair_scale.float().contiguous()
        xc = x.contiguous()                    # referenced until the launch is enqueued
        L.check(L.load().dewb_moe_push(L.ptr(xc), L.ptr(ps), L.ptr(plan.dest_rank), L.ptr(plan.dest_pos), buf.ptr_array(),
                                       None, self.flags.ptr_array(), L.ptr(self.flags.tensor), ctypes.c_int(self.SLOT_READY),
                                       ctypes.c_int(self.SLOT_PUSHED), ctypes.c_uint(self.seq), ctypes.c_ulonglong(self.limit_ns),
                                       L.ptr(self.counter), ctypes.c_int(T), ctypes.c_int(d), ctypes.c_int(plan.top_k), ctypes.c_int(self.rank),
                                       ctypes.c_int(self.world), ctypes.c_int(0), L.ptr(L.status(x.device)), L.stream_ptr()), "moe_push")
        L.count_launches()
        self._wait(self.SLOT_PUSHED, self.seq)
        if not self.lean:
            return buf.tensor[: self.rows_cap * d].view(self.rows_cap, d).clone()
        buf.tensor.view(self.rows_cap + 1, d).index_fill_(0, plan.pad_rows, 0)
        # a tensor of its own over the buffer's memory, not a view: autograd saves it for the weight gradient, and the buffer's next
        # use (the following microbatch's push, after this microbatch's backward) must not read as an in-place change of a saved view
        base = buf.tensor
        return torch.empty(0, dtype=base.dtype, device=base.device).set_(base.untyped_storage(), base.storage_offset(), (self.rows_cap, d), (d, 1))

    def claim_out(self, d: int) -> torch.Tensor:
        """The buffer the peers pull from, once nobody reads its previous contents any more: a producer that writes the rows there
        (and passes this very tensor to ``pull``) saves the copy."""
        if self.last_pull:
            self._wait(self.SLOT_PULLED, self.last_pull)
        self._out_claimed = True
        # a tensor of its own over the buffer's memory (not a view: what is written there has no autograd history to join)
        base = self.out.tensor
        return torch.empty(0, dtype=base.dtype, device=base.device).set_(base.untyped_storage(), base.storage_offset(), (self.rows_cap, d), (d, 1))

    def pull(self, rows: torch.Tensor, plan: ExchangePlan, weights: Optional[torch.Tensor] = None, keep_rows: bool = False):
        """``rows [rows_cap, d]`` on every owner -> ``out [T, d]``: each token's k rows, weighted and summed (fp32 accumulate)."""
        d = rows.shape[1]
        T, k = plan.tokens, plan.top_k
        L.ensure_device(rows)
        self.seq += 1
        in_place = self._out_claimed and rows.data_ptr() == self.out.tensor.data_ptr()
        if not in_place:
            if self.last_pull and not self._out_claimed:
                self._wait(self.SLOT_PULLED, self.last_pull)          # nobody still reads the previous contents of `out`
            self.out.tensor.view(self.rows_cap, d).copy_(rows)
        self._out_claimed = False
        self._signal(self.SLOT_OUT)
        out = torch.empty(T, d, dtype=torch.bfloat16, device=rows.device)
        gathered = torch.empty(T * k, d, dtype=torch.bfloat16, device=rows.device) if keep_rows else None
        w = None if weights is None else weights.float().contiguous()
        L.check(L.load().dewb_moe_pull(self.out.ptr_array(), L.ptr(w), L.ptr(plan.dest_rank), L.ptr(plan.dest_pos), L.ptr(out), L.ptr(gathered),
                                       self.flags.ptr_array(), L.ptr(self.flags.tensor), ctypes.c_int(self.SLOT_OUT), ctypes.c_int(self.SLOT_PULLED),
                                       ctypes.c_uint(self.seq), ctypes.c_ulonglong(self.limit_ns), L.ptr(self.counter[1:]), ctypes.c_int(T),
                                       ctypes.c_int(d), ctypes.c_int(k), ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                       L.ptr(L.status(rows.device)), L.stream_ptr()), "moe_pull")
        L.count_launches()
        self.last_pull = self.seq
        return out, gathered


class _PushRows(torch.autograd.Function):
    """Dispatch; its backward is a combine with unit weights (the sum of a token's k row gradients)."""

    @staticmethod
    def forward(ctx, x, exchange, plan):
        ctx.exchange, ctx.plan = exchange, plan
        return exchange.push(x, plan)

    @staticmethod
    def backward(ctx, d_rows):
        dx, _ = ctx.exchange.pull(d_rows.contiguous(), ctx.plan, None)
        return dx, None, None


class _PullRows(torch.autograd.Function):
    """Combine; its backward dispatches ``w[t, j] * dy[t]`` to the owners and takes ``dw[t, j] = <dy[t], row(t, j)>``."""

    @staticmethod
    def forward(ctx, rows, weights, exchange, plan):
        ctx.exchange, ctx.plan = exchange, plan
        out, gathered = exchange.pull(rows, plan, weights, keep_rows=weights.requires_grad)
        ctx.save_for_backward(weights, gathered)
        return out

    @staticmethod
    def backward(ctx, dy):
        weights, gathered = ctx.saved_tensors
        plan = ctx.plan
        dy = dy.contiguous()
        d_rows = ctx.exchange.push(dy, plan, pair_scale=weights.reshape(-1), backward=True)
        dw = None
        if gathered is not None:
            dw = (gathered.view(plan.tokens, plan.top_k, -1).float() * dy.float().unsqueeze(1)).sum(-1).to(weights.dtype)
        return d_rows, dw, None, None


def exchange_experts(exchange: TokenExchange, experts, x2: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """plan -> dispatch -> grouped expert MLP on the received rows -> combine, all on this library's kernels."""
    plan = exchange.plan(ids, x2.shape[1])
    exchange.last_info = plan.info            # device tensor {rows received, overflowed, busiest owner's rows, pairs dropped}: read it after the step
    if getattr(exchange, "totals", None) is None:
        exchange.totals = torch.zeros(3, dtype=torch.int64, device=x2.device)      # {calls overflowed, pairs dropped, busiest owner's rows ever}
    with torch.no_grad():
        exchange.totals[:2] += plan.info[[1, 3]]
        exchange.totals[2] = torch.maximum(exchange.totals[2], plan.info[2].long())
    rows = _PushRows.apply(x2, exchange, plan)
    if exchange.lean:
        out_rows = experts(rows, plan.layout, out=exchange.claim_out(x2.shape[1]) if exchange.write_in_place else None, lean=True)
    else:
        out_rows = experts(rows, plan.layout)
    return _PullRows.apply(out_rows, weights.float(), exchange, plan)


class _GatherExperts(torch.autograd.Function):
    """All-gather of a rank's expert slice ``[E / W, ...]`` along the expert axis -> ``[E, ...]``; the backward is a
    reduce-scatter (sum) of the full gradient, so every owner receives its experts' gradient from all ranks' tokens."""

    @staticmethod
    def forward(ctx, w, group):
        ctx.group = group
        W = dist.get_world_size(group)
        out = w.new_empty((W * w.shape[0],) + tuple(w.shape[1:]))
        dist.all_gather_into_tensor(out, w.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        W = dist.get_world_size(ctx.group)
        mine = g.new_empty((g.shape[0] // W,) + tuple(g.shape[1:]))
        if g.dtype == torch.bfloat16 and not g.is_cuda:
            gf = g.float().contiguous()
            mf = gf.new_empty(mine.shape)
            dist.reduce_scatter_tensor(mf, gf, group=ctx.group)
            mine = mf.to(g.dtype)
        else:
            dist.reduce_scatter_tensor(mine, g.contiguous(), group=ctx.group)
        return mine, None


class ExpertParallel:
    def __init__(self, group: Optional[dist.ProcessGroup] = None, fused: bool = True, capacity_factor: Optional[float] = None):
        # rows an owner's receive buffer holds, as a multiple of one rank's (token, choice) pairs: `world` can never overflow;
        # pairs past the end are dropped and counted (DEWB_EP_CAPACITY overrides the default of 2)
        if capacity_factor is None:
            capacity_factor = float(os.environ.get("DEWB_EP_CAPACITY", "2.0"))
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.fused, self.capacity_factor = fused, capacity_factor
        self.exchange: Optional[TokenExchange] = None        # one set of symmetric buffers shared by every sparse layer

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

    # ------------------------------------------------------------------ dispatch='global': weights travel, tokens stay
    def gathered_experts(self, mlp, x2: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """``dispatch='global'``: every rank all-gathers the experts' weights along the expert axis and runs all experts on
        its own tokens; the backward reduce-scatters the weight gradients back to their owners.  It moves
        ``3 d F E (W - 1) / W`` weight elements per layer instead of ``2 k d`` per token, so it wins when a rank's tokens
        outnumber ``1.5 F E / k`` (reference: ``Gathered`` / ``dispatch='global'``, src/dew/nn/moe.py:648,858-930)."""
        T, k = ids.shape
        gate_up = _GatherExperts.apply(mlp.experts.gate_up, self.group)
        down = _GatherExperts.apply(mlp.experts.down, self.group)
        layout = G.group_layout(ids, mlp.mix.experts)
        xs = G.permute(x2, layout, k)
        h = G.grouped_linear(xs, gate_up, layout)
        from .. import ops
        ys = G.grouped_linear(ops.packed_swiglu(h), down, layout)
        return G.combine(ys, layout, weights.to(x2.dtype) if x2.dtype != torch.float32 else weights, T)

    # ------------------------------------------------------------------ the exchange
    def dispatch_compute_combine(self, mlp, x2: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        if getattr(mlp.mix, "dispatch", "auto") == "global" and self.world > 1:
            return self.gathered_experts(mlp, x2, weights, ids)
        if x2.is_cuda and x2.dtype == torch.bfloat16 and L.use_cuda(x2) and self.fused:
            # device-planned exchange over peer memory (TokenExchange); the path below is the NCCL / gloo form of the same protocol
            if self.exchange is None:
                self.exchange = TokenExchange(mlp.mix.experts, self.group, self.capacity_factor)
            return exchange_experts(self.exchange, mlp.experts, x2, weights, ids)
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
