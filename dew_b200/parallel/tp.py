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
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import library as L
from .symm import SymmetricBuffer


class TensorParallel:
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
        if self.fused:
            self.buf = SymmetricBuffer(2 * max_rows * features, torch.bfloat16, self.device, group, zero=True)
            self.flags = SymmetricBuffer(64, torch.int32, self.device, group, zero=True)
            self.counters = torch.zeros(4, dtype=torch.int32, device=self.device)    # {sequence, arrive, leave}

    # ------------------------------------------------------------------ inference path (no autograd)
    def reduce_add_norm(self, partial: torch.Tensor, residual: Optional[torch.Tensor], norm_w: Optional[torch.Tensor],
                        eps: float = 1e-6) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
        """``h = residual + sum_ranks(partial)``; returns ``(norm(h) * w or None, h)``."""
        shape = partial.shape
        d = shape[-1]
        p2 = partial.reshape(-1, d)
        rows = p2.shape[0]
        if self.world == 1:
            h = p2 if residual is None else (p2.float() + residual.reshape(-1, d).float()).to(p2.dtype)
            n = ops.rms_norm(h, norm_w, eps) if norm_w is not None else None
            return (None if n is None else n.reshape(shape)), h.reshape(shape)
        if not self.fused or rows > self.max_rows or d != self.features or p2.dtype != torch.bfloat16:
            s = p2.float().contiguous()
            dist.all_reduce(s, group=self.group)
            h = (s if residual is None else s + residual.reshape(-1, d).float()).to(p2.dtype)
            n = ops.rms_norm_reference(h, norm_w, eps) if norm_w is not None else None
            return (None if n is None else n.reshape(shape)), h.reshape(shape)
        h = torch.empty((rows, d), dtype=torch.bfloat16, device=self.device)
        n = torch.empty_like(h) if norm_w is not None else None
        res = residual.reshape(-1, d).contiguous() if residual is not None else None
        L.check(L.load().dewb_allreduce_rows(self.buf.ptr_array(), self.flags.ptr_array(), L.ptr(p2.contiguous()), L.ptr(res),
                                             L.ptr(norm_w.to(torch.bfloat16) if norm_w is not None else None), L.ptr(h), L.ptr(n),
                                             ctypes.c_int(rows), ctypes.c_int(d), ctypes.c_float(eps), ctypes.c_int(self.rank),
                                             ctypes.c_int(self.world), L.ptr(self.counters),
                                             ctypes.c_longlong(self.max_rows * self.features), ctypes.c_int(0),
                                             ctypes.c_ulonglong(self.limit_ns), L.ptr(L.status(self.device)), L.stream_ptr()),
                "allreduce_rows")
        L.count_launches()
        return (None if n is None else n.reshape(shape)), h.reshape(shape)

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


def tensor_parallelize(model, tp: TensorParallel):
    """Shard a ``CausalTransformer`` in place over ``tp``'s group. Heads, KV heads, MLP width and vocabulary must
    divide by the group size."""
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
        model.tp_head = nn.Parameter(_shard_rows(head_w, r, W), requires_grad=False)
        if model.head is not None:
            model.head = None
            model.config.tie_embeddings = True      # the full head is gone; logits come from `tp_head`
    model.tp = tp
    model.local_kv_heads = Hkv // W
    return model
