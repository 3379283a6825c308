"""Tensor parallelism: Megatron-style split of attention heads, MLP columns and the vocabulary over the ``tensor`` axis.

* Column-parallel projections (QKV, gate|up, head) keep their rows' shard; row-parallel projections (attention output,
  MLP down) keep their columns' shard and produce partial sums.
* The partial sums are combined by this library's own one-shot all-reduce over peer memory, fused with the residual
  add and the next RMSNorm (``dewb_allreduce_rows``) - one kernel where a stock stack runs NCCL all-reduce + add +
  norm.  On CPU ranks (gloo) or one process the same arithmetic runs through ``torch.distributed``.
* For training, ``copy_to_region`` / ``reduce_from_region`` are the autograd-aware conjugate pair (identity forward +
  all-reduce backward, and the reverse).

Reference behaviour: ``mlp / heads / kv / vocab -> tensor`` rules (src/dew/mesh.py:101-146; src/dew/nn/sharding.py:76-99),
serving with heads split over ``tensor`` (src/dew/inference/serving.py:179).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import library as L
from .symm import SymmetricBuffer


class TensorParallel:
    REGIONS = 4
    LL_ROWS = 512

    def __init__(self, group: Optional[dist.ProcessGroup] = None, max_rows: int = 4096, features: int = 4096,
                 device=None, wait_limit_s: float = 20.0):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.max_rows, self.features = max_rows, features
        self.limit_ns = int(wait_limit_s * 1e9)
        self.seq = 0
        self.fused = self.device.type == "cuda" and self.world > 1
        # How the fused all-reduce + add + norm moves its rows (DEWB_TP_ALLREDUCE):
        #   'auto' (default)  up to LL_ROWS rows take the low-latency kernel (every 16-byte store carries its own arrival flag,
        #                     ordinary local outputs); more rows take the two-shot kernel below
        #   'twoshot'         rows are pushed to their owners, reduced there and pushed back; a flag per phase; outputs in
        #                     peer-visible memory
        #   'oneshot'         every rank pulls every peer's whole partial (the earlier form, kept for comparison)
        self.mode = os.environ.get("DEWB_TP_ALLREDUCE", "auto")
        if self.mode not in ("auto", "ll", "twoshot", "oneshot"):
            raise ValueError(f"DEWB_TP_ALLREDUCE must be auto, ll, twoshot or oneshot, not {self.mode!r}")
        self.calls = 0
        if self.fused:
            self.flags = SymmetricBuffer(64, torch.int32, self.device, group, zero=True)
            # one-shot {sequence, arrive, leave, -}; two-shot {sequence, ticket 1, ticket 2, -}; low-latency {sequence, leave}
            self.counters = torch.zeros(12, dtype=torch.int32, device=self.device)
            if self.mode == "oneshot":
                self.buf = SymmetricBuffer(2 * max_rows * features, torch.bfloat16, self.device, group, zero=True)
            else:
                # per region: slots [world][ceil(max_rows / world)][d] | sum [max_rows][d] | norm [max_rows][d]; regions alternate
                # from call to call, so an output stays valid until REGIONS - 1 further calls have been made
                self.owner_rows = -(-max_rows // self.world)
                self.region = (self.world * self.owner_rows + 2 * max_rows) * features
                self.buf = SymmetricBuffer(self.REGIONS * self.region, torch.bfloat16, self.device, group, zero=True)
            if self.mode in ("auto", "ll"):
                # line format: 4 bytes per element; per region: slots [world][ceil(ll_rows / world)][d] | sums [ll_rows][d]
                self.ll_rows = min(max_rows, self.LL_ROWS) if self.mode == "auto" else max_rows
                self.ll_owner_rows = -(-self.ll_rows // self.world)
                self.ll_region = (self.world * self.ll_owner_rows + self.ll_rows) * features * 4
                self.ll_buf = SymmetricBuffer(2 * self.ll_region // 4, torch.int32, self.device, group, zero=True)

    # ------------------------------------------------------------------ inference path (no autograd)
    def reduce_add_norm(self, partial: torch.Tensor, residual: Optional[torch.Tensor], norm_w: Optional[torch.Tensor],
                        eps: float = 1e-6) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
        """``h = residual + sum_ranks(partial)``; returns ``(norm(h) * w or None, h)``."""
        shape = partial.shape
        d = shape[-1]
        p2 = partial.reshape(-1, d)
        rows = p2.shape[0]
        if self.world == 1:
            if residual is not None and norm_w is not None:
                n, h = ops.stream_rms_norm(residual.reshape(-1, d), p2, norm_w, eps)      # add + norm in one kernel
                return n.reshape(shape), h.reshape(shape)
            h = p2 if residual is None else (p2.float() + residual.reshape(-1, d).float()).to(p2.dtype)
            n = ops.rms_norm(h, norm_w, eps) if norm_w is not None else None
            return (None if n is None else n.reshape(shape)), h.reshape(shape)
        if self.fused and rows > self.max_rows and d == self.features and p2.dtype == torch.bfloat16:
            # more rows than the peer-visible buffers hold: the fused kernel block by block, results gathered into one tensor
            h = torch.empty((rows, d), dtype=torch.bfloat16, device=self.device)
            n = torch.empty_like(h) if norm_w is not None else None
            res2 = residual.reshape(-1, d) if residual is not None else None
            for r0 in range(0, rows, self.max_rows):
                r1 = min(rows, r0 + self.max_rows)
                nb, hb = self.reduce_add_norm(p2[r0:r1], None if res2 is None else res2[r0:r1], norm_w, eps)
                h[r0:r1].copy_(hb)
                if n is not None:
                    n[r0:r1].copy_(nb)
            return (None if n is None else n.reshape(shape)), h.reshape(shape)
        if not self.fused or rows > self.max_rows or d != self.features or p2.dtype != torch.bfloat16:
            s = p2.float().contiguous()
            dist.all_reduce(s, group=self.group)
            h = (s if residual is None else s + residual.reshape(-1, d).float()).to(p2.dtype)
            n = ops.rms_norm_reference(h, norm_w, eps) if norm_w is not None else None
            return (None if n is None else n.reshape(shape)), h.reshape(shape)
        if self.mode in ("auto", "ll") and rows <= self.ll_rows:
            return self._low_latency(p2, residual, norm_w, eps, shape)
        if self.mode != "oneshot":
            return self._two_shot(p2, residual, norm_w, eps, shape)
        h = torch.empty((rows, d), dtype=torch.bfloat16, device=self.device)
        n = torch.empty_like(h) if norm_w is not None else None
        res = residual.reshape(-1, d).contiguous() if residual is not None else None
        pc = p2.contiguous()                                         # both referenced until the launch is enqueued
        wc = norm_w.to(torch.bfloat16) if norm_w is not None else None
        L.check(L.load().dewb_allreduce_rows(self.buf.ptr_array(), self.flags.ptr_array(), L.ptr(pc), L.ptr(res),
                                             L.ptr(wc), L.ptr(h), L.ptr(n),
                                             ctypes.c_int(rows), ctypes.c_int(d), ctypes.c_float(eps), ctypes.c_int(self.rank),
                                             ctypes.c_int(self.world), L.ptr(self.counters),
                                             ctypes.c_longlong(self.max_rows * self.features), ctypes.c_int(0),
                                             ctypes.c_ulonglong(self.limit_ns), L.ptr(L.status(self.device)), L.stream_ptr()),
                "allreduce_rows")
        L.count_launches()
        return (None if n is None else n.reshape(shape)), h.reshape(shape)

    def _low_latency(self, p2, residual, norm_w, eps, shape):
        rows, d = p2.shape
        base = (self.calls & 1) * self.ll_region
        self.calls += 1
        # the row geometry of the call (not of the buffer) places the slots, so both offsets depend on this call's rows only
        owner_rows = -(-rows // self.world)
        sums_off = base + self.world * owner_rows * d * 4
        h = torch.empty((rows, d), dtype=torch.bfloat16, device=self.device)
        n = torch.empty_like(h) if norm_w is not None else None
        res = residual.reshape(-1, d).contiguous() if residual is not None else None
        pc = p2.contiguous()                                         # all referenced until the launch is enqueued
        wc = norm_w.to(torch.bfloat16) if norm_w is not None else None
        L.check(L.load().dewb_allreduce_rows_ll(self.ll_buf.ptr_array(), L.ptr(pc), L.ptr(res), L.ptr(wc), L.ptr(h), L.ptr(n),
                                                ctypes.c_int(rows), ctypes.c_int(d), ctypes.c_float(eps), ctypes.c_int(self.rank),
                                                ctypes.c_int(self.world), L.ptr(self.counters[8:]), ctypes.c_longlong(base),
                                                ctypes.c_longlong(sums_off), ctypes.c_ulonglong(self.limit_ns),
                                                L.ptr(L.status(self.device)), L.stream_ptr()), "allreduce_rows_ll")
        L.count_launches()
        return (None if n is None else n.reshape(shape)), h.reshape(shape)

    def _two_shot(self, p2, residual, norm_w, eps, shape):
        """The two-shot kernel.  The returned tensors are views of this object's peer-visible buffer: they stay valid until
        ``REGIONS - 1`` further calls have been made (a decoder layer consumes them before its next call); clone to keep longer."""
        rows, d = p2.shape
        base = (self.calls % self.REGIONS) * self.region
        self.calls += 1
        slots_off = base
        sum_off = base + self.world * self.owner_rows * d
        norm_off = sum_off + self.max_rows * d
        res = residual.reshape(-1, d).contiguous() if residual is not None else None
        pc = p2.contiguous()                                         # all referenced until the launch is enqueued
        wc = norm_w.to(torch.bfloat16) if norm_w is not None else None
        L.check(L.load().dewb_allreduce_rows_2shot(self.buf.ptr_array(), self.flags.ptr_array(), L.ptr(pc), L.ptr(res), L.ptr(wc),
                                                   ctypes.c_int(rows), ctypes.c_int(d), ctypes.c_float(eps), ctypes.c_int(self.rank),
                                                   ctypes.c_int(self.world), L.ptr(self.counters[4:]), ctypes.c_longlong(slots_off),
                                                   ctypes.c_longlong(sum_off), ctypes.c_longlong(norm_off), ctypes.c_int(16),
                                                   ctypes.c_ulonglong(self.limit_ns), L.ptr(L.status(self.device)), L.stream_ptr()),
                "allreduce_rows_2shot")
        L.count_launches()
        h = self.buf.tensor[sum_off:sum_off + rows * d].view(shape)
        n = self.buf.tensor[norm_off:norm_off + rows * d].view(shape) if norm_w is not None else None
        return n, h

    def all_reduce(self, partial: torch.Tensor) -> torch.Tensor:
        return self.reduce_add_norm(partial, None, None)[1]

    def argmax_vocab_parallel(self, local_logits: torch.Tensor) -> torch.Tensor:
        """Greedy token from vocabulary-sharded logits ``[R, V / W]`` without gathering the logits."""
        val, idx = local_logits.float().max(-1)
        if self.world == 1:
            return idx
        pair = torch.stack([val, (idx + self.rank * local_logits.shape[-1]).float()], -1).contiguous()
        gathered = [torch.empty_like(pair) for _ in range(self.world)]
        dist.all_gather(gathered, pair, group=self.group)
        allp = torch.stack(gathered, 0)                              # [W, R, 2]
        best = allp[..., 0].argmax(0)                                # [R]
        return allp[best, torch.arange(pair.shape[0], device=pair.device), 1].long()


class SequenceParallelLinear:
    """The two tensor-parallel products of a sequence-parallel region, each ONE kernel that does the product and its
    collective over peer memory (``csrc/kernels/gemm_comm_sm100.cu``):

    * ``gather_matmul(x_shard, w)``: ``all_gather_rows(x) @ w.T`` - A tiles are read from the owning rank's memory by
      TMA while other tiles compute; nothing is gathered first.
    * ``matmul_scatter(x, w, residual_shard)``: ``reduce_scatter_rows(x @ w.T) (+ residual)`` - finished tiles are stored
      into the owner's partial buffer from the epilogue; the owner sums the W slots.

    Row counts are fixed at construction (``rows`` total, a multiple of ``128 * world``).  On CPU ranks, one rank, or
    unfit shapes the same arithmetic runs through ``torch.distributed``.

    Reference: sequence-parallel (``SPREAD``) activations around the Megatron-split projections
    (src/dew/nn/sharding.py:262-280, src/dew/mesh.py:101-146)."""

    def __init__(self, group, rows: int, in_features: int, out_features: int, device=None, wait_limit_s: float = 20.0):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.rows, self.in_features, self.out_features = rows, in_features, out_features
        self.limit_ns = int(wait_limit_s * 1e9)
        self.seq = 0
        self.fused = self.device.type == "cuda" and self.world > 1 and rows % (128 * self.world) == 0
        if self.fused:
            W = self.world
            Ms = rows // W
            # peers read the shard and write the partial slots: both are double-buffered by call parity
            self.x_shard = SymmetricBuffer(2 * Ms * in_features, torch.bfloat16, self.device, group, zero=True)
            self.partials = SymmetricBuffer(2 * W * Ms * out_features, torch.bfloat16, self.device, group, zero=True)
            self.flags = SymmetricBuffer(64, torch.int32, self.device, group, zero=True)
            self.staging = torch.empty((rows, in_features), dtype=torch.bfloat16, device=self.device)
            self.block_ready = torch.zeros(rows // 128, dtype=torch.int32, device=self.device)
            self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.ag_calls = 0
            self.rs_calls = 0

    def shard_buffer(self) -> torch.Tensor:
        """The peer-visible buffer the NEXT ``gather_matmul`` reads this rank's rows from: a producer that writes its
        output here (and passes this very tensor) saves the copy."""
        Ms = self.rows // self.world
        n = Ms * self.in_features
        return self.x_shard.tensor[(self.ag_calls & 1) * n:((self.ag_calls & 1) + 1) * n].view(Ms, self.in_features)

    def gather_matmul(self, x_shard: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``x_shard [rows / W, K]`` (this rank's rows), ``w [N, K]`` -> ``[rows, N]``."""
        W = self.world
        if not self.fused or x_shard.dtype != torch.bfloat16 or x_shard.shape[1] != self.in_features:
            if W == 1:
                return ops.linear(x_shard, w)
            parts = [torch.empty_like(x_shard) for _ in range(W)]
            dist.all_gather(parts, x_shard.contiguous(), group=self.group)
            return ops.linear(torch.cat(parts, 0), w)
        lib = L.load()
        K, N = self.in_features, w.shape[0]
        buf = self.shard_buffer()
        if x_shard.data_ptr() != buf.data_ptr():
            buf.copy_(x_shard)
        parity = self.ag_calls & 1
        self.ag_calls += 1
        out = torch.empty((self.rows, N), dtype=torch.bfloat16, device=self.device)
        L.check(lib.dewb_ag_gemm_bf16(self.x_shard.ptr_array(parity * (self.rows // W) * K * 2), L.ptr(w), L.ptr(out), L.ptr(self.staging),
                                      L.ptr(self.block_ready), ctypes.c_uint(self.ag_calls), ctypes.c_int(self.rows), ctypes.c_int(N),
                                      ctypes.c_int(K), ctypes.c_longlong(K), ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(N),
                                      ctypes.c_int(self.rank), ctypes.c_int(W), self.flags.ptr_array(), L.ptr(self.flags.tensor),
                                      ctypes.c_int(0), ctypes.c_uint(self.ag_calls), ctypes.c_ulonglong(self.limit_ns),
                                      L.ptr(L.status(self.device)), L.stream_ptr()), "ag_gemm")
        L.count_launches()
        return out

    def matmul_scatter(self, x: torch.Tensor, w: torch.Tensor, residual_shard: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x [rows, K_local]``, ``w [N, K_local]`` (this rank's slice of the reduction) -> this rank's rows
        ``[rows / W, N]`` of the summed product (+ ``residual_shard``)."""
        W = self.world
        N = w.shape[0]
        if not self.fused or x.dtype != torch.bfloat16 or N != self.out_features or x.shape[0] != self.rows:
            y = ops.linear(x, w)
            if W > 1:
                full = y.float().contiguous()
                mine = torch.empty((x.shape[0] // W, N), dtype=torch.float32, device=y.device)
                dist.reduce_scatter_tensor(mine, full, group=self.group)
                y = mine.to(x.dtype)
            return y if residual_shard is None else y + residual_shard
        lib = L.load()
        parity = self.rs_calls & 1
        self.rs_calls += 1
        Ms = self.rows // W
        off = parity * W * Ms * N * 2
        L.check(lib.dewb_gemm_rs_bf16(L.ptr(x), L.ptr(w), self.partials.ptr_array(off), ctypes.c_int(self.rows), ctypes.c_int(N),
                                      ctypes.c_int(x.shape[1]), ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(w.stride(0)),
                                      ctypes.c_int(self.rank), ctypes.c_int(W), self.flags.ptr_array(), ctypes.c_int(1),
                                      ctypes.c_uint(self.rs_calls), L.ptr(self.counter), L.ptr(L.status(self.device)), L.stream_ptr()),
                "gemm_rs")
        out = torch.empty((Ms, N), dtype=torch.bfloat16, device=self.device)
        res = residual_shard.contiguous() if residual_shard is not None else None
        mine = self.partials.tensor[parity * W * Ms * N:(parity + 1) * W * Ms * N]
        L.check(lib.dewb_reduce_partials(L.ptr(mine), L.ptr(res), L.ptr(out), ctypes.c_longlong(Ms),
                                         ctypes.c_int(N), ctypes.c_int(W), L.ptr(self.flags.tensor), ctypes.c_int(1),
                                         ctypes.c_uint(self.rs_calls), ctypes.c_ulonglong(self.limit_ns), L.ptr(L.status(self.device)),
                                         L.stream_ptr()), "reduce_partials")
        L.count_launches(2)
        return out


# ------------------------------------------------------------------------------------------------ autograd-aware pair
class _CopyToRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_region(x, group=None):
    return _CopyToRegion.apply(x, group)


def reduce_from_region(x, group=None):
    return _ReduceFromRegion.apply(x, group)


# ------------------------------------------------------------------------------------------------ sharding a model
def _shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n].clone()


def _shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[1] // world
    return w[:, rank * n:(rank + 1) * n].clone()


def tensor_parallelize(model, tp: TensorParallel, training: bool = False):
    """Shard a ``CausalTransformer`` in place over ``tp``'s group. Heads, KV heads, MLP width and vocabulary must
    divide by the group size.  With ``training`` the vocabulary-parallel head is a trainable parameter and the layers run
    the autograd-aware conjugate pair around their sharded products (identity forward / all-reduce backward in front of the
    column-parallel projections, all-reduce forward / identity backward behind the row-parallel ones)."""
    W, r = tp.world, tp.rank
    cfg = model.config
    Hq, Hkv = cfg.num_heads, cfg.num_kv_heads or cfg.num_heads
    D = cfg.head_dim or cfg.emb_features // cfg.num_heads
    if Hq % W or Hkv % W or cfg.vocab_size % W:
        raise ValueError(f"heads {Hq}/{Hkv} and vocabulary {cfg.vocab_size} must divide by the tensor-parallel size {W}")
    with torch.no_grad():
        for layer in model.layers:
            att = layer.mixer
            if hasattr(att, "qkv_proj"):
                w = att.qkv_proj.weight.data
                q, k, v = w[: Hq * D], w[Hq * D:(Hq + Hkv) * D], w[(Hq + Hkv) * D:]
                att.qkv_proj.weight = nn.Parameter(torch.cat([_shard_rows(q, r, W), _shard_rows(k, r, W), _shard_rows(v, r, W)], 0),
                                                   requires_grad=att.qkv_proj.weight.requires_grad)
                b = att.qkv_proj.bias
                if b is not None:                          # column-parallel: each rank keeps the bias of its own heads
                    bq, bk, bv = b.data[: Hq * D], b.data[Hq * D:(Hq + Hkv) * D], b.data[(Hq + Hkv) * D:]
                    att.qkv_proj.bias = nn.Parameter(torch.cat([_shard_rows(bq, r, W), _shard_rows(bk, r, W), _shard_rows(bv, r, W)], 0),
                                                     requires_grad=b.requires_grad)
                    att.qkv_proj.bias.tensor_parallel = True
                if att.o_proj.bias is not None:
                    raise ValueError("a bias on the row-parallel output projection would be added once per rank; fold it away before sharding")
                att.o_proj.weight = nn.Parameter(_shard_cols(att.o_proj.weight.data, r, W), requires_grad=att.o_proj.weight.requires_grad)
                att.num_heads, att.num_kv_heads = Hq // W, Hkv // W
            mlp = layer.mlp
            if hasattr(mlp, "gate_up_proj"):
                w = mlp.gate_up_proj.weight.data
                F_ = w.shape[0] // 2
                if F_ % W:
                    raise ValueError(f"MLP width {F_} must divide by the tensor-parallel size {W}")
                mlp.gate_up_proj.weight = nn.Parameter(torch.cat([_shard_rows(w[:F_], r, W), _shard_rows(w[F_:], r, W)], 0),
                                                       requires_grad=mlp.gate_up_proj.weight.requires_grad)
                mlp.down_proj.weight = nn.Parameter(_shard_cols(mlp.down_proj.weight.data, r, W), requires_grad=mlp.down_proj.weight.requires_grad)
                mlp.hidden = F_ // W
            layer.tp = tp
        head_w = model.head_weight().data
        model.tp_head = nn.Parameter(_shard_rows(head_w, r, W), requires_grad=training)
        if training:
            for attr in ("logical_axes", "dew_kind"):
                src = model.head.weight if model.head is not None else model.embed.weight
                if hasattr(src, attr):
                    setattr(model.tp_head, attr, getattr(src, attr))
            model.tp_head.dew_kind = "kernel"
        if model.head is not None:
            model.head = None
            model.config.tie_embeddings = True      # the full head is gone; logits come from `tp_head`
    for layer in model.layers:
        for mod, names in ((layer.mixer, ("qkv_proj", "o_proj")), (layer.mlp, ("gate_up_proj", "down_proj"))):
            for nm in names:
                lin = getattr(mod, nm, None)
                if lin is not None:
                    lin.weight.tensor_parallel = True          # this rank's slice: other tensor ranks hold the other slices
    model.tp_head.tensor_parallel = True
    model.tp = tp
    model.tp_training = training
    for layer in model.layers:
        layer.tp_training = training
    model.local_kv_heads = Hkv // W
    return model
