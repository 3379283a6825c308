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


class Variants:
    """The optional attention variants the kernels take: ``window`` (keys visible behind each query, None = all), ``softcap``
    (scores become cap * tanh(score / cap)), ``sinks`` ([Hq] fp32 logits that join the softmax denominator only) and
    ``segments`` (int32 [B, S] ids of packed documents, non-decreasing along the sequence; 0 marks padding)."""

    def __init__(self, window=None, softcap: float = 0.0, sinks=None, segments=None):
        self.window = int(window) if window else 0
        self.softcap = float(softcap or 0.0)
        self.sinks = sinks.detach().to(torch.float32).contiguous() if sinks is not None else None
        self.segments = segments.to(torch.int32).contiguous() if segments is not None else None

    def any(self) -> bool:
        return bool(self.window or self.softcap or self.sinks is not None or self.segments is not None)


NONE = Variants()


def flash_fwd(q, k, v, causal: bool, scale: float, need_lse: bool = True, var: Variants = NONE):
    B, S, Hq, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    out = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device) if need_lse else None
    rc = L.load().dewb_flash_fwd_var(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(out), L.ptr(lse), c_int(B), c_int(S), c_int(T),
                                     c_int(Hq), c_int(Hkv), c_int(D), *_strides(q), *_strides(k), *_strides(v),
                                     *_strides(out), c_float(scale), c_int(int(causal)), c_int(var.window), c_float(var.softcap),
                                     L.ptr(var.sinks), L.ptr(var.segments), L.ptr(var.segments), L.ptr(L.status(q.device)),
                                     L.stream_ptr())
    L.check(rc, "flash_fwd")
    L.count_launches()
    return out, lse


def bwd_available() -> bool:
    try:
        return hasattr(L.load(), "dewb_flash_bwd")
    except Exception:
        return False


def flash_bwd(do, q, k, v, out, lse, causal: bool, scale: float, grads=None, var: Variants = NONE, want_delta: bool = False):
    """dq, dk, dv.  ``grads`` may supply the three output tensors (e.g. views of one fused ``[B, S, H + 2 Hkv, D]``
    gradient buffer); any strides with a unit stride along D and 16-byte aligned rows are taken as they are."""
    B, S, Hq, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    if grads is None:
        dq = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, T, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((B, T, Hkv, D), dtype=q.dtype, device=q.device)
    else:
        dq, dk, dv = grads
    delta = torch.empty((2, B, Hq, S), dtype=torch.float32, device=q.device)     # delta, then lse in log2 units
    if do.stride(3) != 1 or any(st % 8 for st in do.stride()[:3]):
        do = do.contiguous()
    st = []
    for t in (q, k, v, out, do, dq, dk, dv):
        assert t.stride(3) == 1
        st += [t.stride(0), t.stride(1), t.stride(2)]
    strides = (c_ll * 24)(*st)
    rc = L.load().dewb_flash_bwd_var(L.ptr(do), L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(out), L.ptr(lse), L.ptr(delta), L.ptr(dq),
                                     L.ptr(dk), L.ptr(dv), c_int(B), c_int(S), c_int(T), c_int(Hq), c_int(Hkv), c_int(D),
                                     strides, c_float(scale), c_int(int(causal)), c_int(var.window), c_float(var.softcap),
                                     L.ptr(var.segments), L.ptr(var.segments), L.ptr(L.status(q.device)), L.stream_ptr())
    L.check(rc, "flash_bwd")
    L.count_launches(3)
    if want_delta:
        return dq, dk, dv, delta[0]
    return dq, dk, dv


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, var, sinks):
        out, lse = flash_fwd(q, k, v, causal, scale, var=var)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale, ctx.var = causal, scale, var
        ctx.sinks_grad = sinks is not None and sinks.requires_grad
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        var = ctx.var
        if ctx.sinks_grad:
            dq, dk, dv, delta = flash_bwd(do, q, k, v, out, lse, ctx.causal, ctx.scale, var=var, want_delta=True)
            # the sink's probability in every row is exp(sink - lse); its value column is zero, so its logit gradient is
            # -p_sink * delta, summed over batch and rows
            p_sink = torch.exp(var.sinks.to(lse.dtype)[None, :, None] - lse)
            dsinks = -(p_sink * delta).sum((0, 2))
            return dq, dk, dv, None, None, None, dsinks
        dq, dk, dv = flash_bwd(do, q, k, v, out, lse, ctx.causal, ctx.scale, var=var)
        return dq, dk, dv, None, None, None, None


def flash_sm100(q, k, v, causal: bool, scale: float, window=None, softcap: float = 0.0, sinks=None, segment_ids=None):
    var = Variants(window, softcap, sinks, segment_ids)
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad or (sinks is not None and sinks.requires_grad)):
        return _Flash.apply(q, k, v, causal, scale, var, sinks)
    return flash_fwd(q, k, v, causal, scale, need_lse=False, var=var)[0]


class _PackedRopeFlash(torch.autograd.Function):
    """RoPE + flash attention over one packed projection ``qkv [B, S, Hq + 2 Hkv, D]``.

    The rotation is applied in place on ``qkv`` (the producing projection does not keep its output), q / k / v are
    views of it, and the backward writes dq / dk / dv straight into one packed gradient buffer on which the inverse
    rotation then runs in place - so neither direction makes a copy, a zero-fill or an add for the three slices."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, Hq, Hkv, causal, scale):
        B, S, H, D = qkv.shape
        pos = None
        if cos is not None:
            if positions is not None:
                pos = positions.reshape(-1).to(torch.int32).contiguous()
            elif B > 1:
                pos = torch.arange(S, device=qkv.device, dtype=torch.int32).repeat(B)
            L.check(L.load().dewb_rope(L.ptr(qkv), L.ptr(cos), L.ptr(sin), L.ptr(pos), c_ll(B * S), c_int(H), c_int(Hq + Hkv),
                                       c_int(D), c_int(cos.shape[0]), c_float(1.0), L.stream_ptr()), "rope")
            L.count_launches()      # written through the raw pointer: autograd neither sees nor needs to see the change
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        out, lse = flash_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(qkv, out, lse, cos, sin, pos)
        ctx.meta = (Hq, Hkv, causal, scale)
        return out

    @staticmethod
    def backward(ctx, do):
        qkv, out, lse, cos, sin, pos = ctx.saved_tensors
        Hq, Hkv, causal, scale = ctx.meta
        B, S, H, D = qkv.shape
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        dqkv = torch.empty_like(qkv)
        flash_bwd(do, q, k, v, out, lse, causal, scale, grads=(dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]))
        if cos is not None:
            L.check(L.load().dewb_rope(L.ptr(dqkv), L.ptr(cos), L.ptr(sin), L.ptr(pos), c_ll(B * S), c_int(H), c_int(Hq + Hkv),
                                       c_int(D), c_int(cos.shape[0]), c_float(-1.0), L.stream_ptr()), "rope_bwd")
            L.count_launches()
        return dqkv, None, None, None, None, None, None, None


def packed_rope_flash(qkv, cos, sin, positions, Hq: int, Hkv: int, causal: bool, scale: float):
    """``qkv`` must be a fresh contiguous bf16 tensor nobody else reads: it is rotated in place."""
    return _PackedRopeFlash.apply(qkv, cos, sin, positions, Hq, Hkv, causal, scale)
