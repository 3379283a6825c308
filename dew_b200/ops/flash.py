"""Python front of the sm_100a flash attention kernels (csrc/kernels/flash_fwd_sm100.cu, flash_bwd_sm100.cu)."""
from __future__ import annotations

import ctypes

import torch

from . import library as L

c_ll, c_int, c_float = ctypes.c_longlong, ctypes.c_int, ctypes.c_float


def _strides(t):
    """(batch, sequence, head) element strides of a [B, L, H, D] tensor with unit stride along D."""
    assert t.stride(3) == 1
    return c_ll(t.stride(0)), c_ll(t.stride(1)), c_ll(t.stride(2))


def flash_fwd(q, k, v, causal: bool, scale: float, need_lse: bool = True):
    B, S, Hq, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    out = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device) if need_lse else None
    rc = L.load().dewb_flash_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(out), L.ptr(lse), c_int(B), c_int(S), c_int(T),
                                 c_int(Hq), c_int(Hkv), c_int(D), *_strides(q), *_strides(k), *_strides(v),
                                 *_strides(out), c_float(scale), c_int(int(causal)), L.ptr(L.status(q.device)),
                                 L.stream_ptr())
    L.check(rc, "flash_fwd")
    L.count_launches()
    return out, lse


def bwd_available() -> bool:
    try:
        return hasattr(L.load(), "dewb_flash_bwd")
    except Exception:
        return False


def flash_bwd(do, q, k, v, out, lse, causal: bool, scale: float):
    B, S, Hq, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    dq = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
    dk = torch.empty((B, T, Hkv, D), dtype=q.dtype, device=q.device)
    dv = torch.empty((B, T, Hkv, D), dtype=q.dtype, device=q.device)
    delta = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    if not do.is_contiguous():
        do = do.contiguous()
    rc = L.load().dewb_flash_bwd(L.ptr(do), L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(out), L.ptr(lse), L.ptr(delta), L.ptr(dq),
                                 L.ptr(dk), L.ptr(dv), c_int(B), c_int(S), c_int(T), c_int(Hq), c_int(Hkv), c_int(D),
                                 *_strides(q), *_strides(k), *_strides(v), *_strides(out), c_float(scale),
                                 c_int(int(causal)), L.ptr(L.status(q.device)), L.stream_ptr())
    L.check(rc, "flash_bwd")
    L.count_launches(3)
    return dq, dk, dv


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        out, lse = flash_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = flash_bwd(do, q, k, v, out, lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


def flash_sm100(q, k, v, causal: bool, scale: float):
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _Flash.apply(q, k, v, causal, scale)
    return flash_fwd(q, k, v, causal, scale, need_lse=False)[0]
