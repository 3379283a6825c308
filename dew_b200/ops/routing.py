"""Router scores and top-k selection on the GPU: one warp per token (``moe_route_kernel``, csrc/kernels/moe_sm100.cu).

The kernel gives the scores ``[T, E]`` (softmax or sigmoid of the fp32 logits), the ``k`` selected experts per token (by
score + selection bias) and their weights (optionally normalised over the k, times ``scaling``).  The gradient flows to
the logits through the weights and through the scores (the balance loss reads them); it is taken by differentiating the
same formula on the saved logits and ids.  Capability: src/dew/nn/moe.py ``Router`` (:316-586).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import library as L


def _formula(logits, ids, score_function: str, norm: bool, scaling: float):
    scores = torch.softmax(logits, -1) if score_function == "softmax" else torch.sigmoid(logits)
    w = scores.gather(-1, ids)
    if norm:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return w * scaling, scores


class _Route(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, k, score_function, norm, scaling):
        T, E = logits.shape
        logits = logits.contiguous()
        scores = torch.empty_like(logits)
        w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
        ids = torch.empty(T, k, dtype=torch.int32, device=logits.device)
        L.ensure_device(logits)
        rc = L.load().dewb_moe_route(L.ptr(logits), L.ptr(bias), L.ptr(scores), L.ptr(w), L.ptr(ids), ctypes.c_int(T), ctypes.c_int(E),
                                     ctypes.c_int(k), ctypes.c_int(int(score_function != "softmax")), ctypes.c_int(int(bool(norm))),
                                     ctypes.c_float(scaling), L.stream_ptr())
        L.check(rc, "moe_route")
        L.count_launches()
        ids = ids.long()
        ctx.save_for_backward(logits, ids)
        ctx.cfg = (score_function, norm, scaling)
        ctx.mark_non_differentiable(ids)
        return w, ids, scores

    @staticmethod
    def backward(ctx, dw, _dids, dscores):
        logits, ids = ctx.saved_tensors
        with torch.enable_grad():
            lg = logits.detach().requires_grad_(True)
            w, scores = _formula(lg, ids, *ctx.cfg)
            grads = [g for g in (dw, dscores)]
            outs = [o for o, g in zip((w, scores), grads) if g is not None]
            gs = [g for g in grads if g is not None]
            (dl,) = torch.autograd.grad(outs, lg, gs) if outs else (torch.zeros_like(lg),)
        return dl, None, None, None, None, None


def route(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int, score_function: str = "softmax", norm: bool = False,
          scaling: float = 1.0):
    """``logits [T, E]`` fp32 -> (weights ``[T, k]`` fp32, ids ``[T, k]`` int64, scores ``[T, E]`` fp32)."""
    if logits.is_cuda and L.use_cuda(logits):
        b = None if bias is None else bias.float().contiguous()
        return _Route.apply(logits.float(), b, k, score_function, bool(norm), float(scaling))
    scores = torch.softmax(logits, -1) if score_function == "softmax" else torch.sigmoid(logits)
    select = scores + bias if bias is not None else scores
    _, ids = torch.topk(select, k, dim=-1)
    w, _ = _formula(logits, ids, score_function, norm, scaling)
    return w, ids, scores
