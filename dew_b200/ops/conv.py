"""Python front of the short causal convolution kernels (csrc/kernels/short_conv.cu)."""
from __future__ import annotations

import ctypes

import torch

from . import library as L


class _ShortConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, act):
        B, T, C = x.shape
        K = w.shape[1]
        wf = w.float().contiguous()
        bf = bias.float().contiguous() if bias is not None else None
        y = torch.empty_like(x)
        L.check(L.load().dewb_short_conv_fwd(L.ptr(x), L.ptr(wf), L.ptr(bf), L.ptr(y), ctypes.c_int(B), ctypes.c_int(T),
                                             ctypes.c_int(C), ctypes.c_int(K), ctypes.c_int(int(act)), L.stream_ptr()), "short_conv_fwd")
        L.count_launches()
        ctx.save_for_backward(x, wf, bf)
        ctx.act, ctx.w_dtype, ctx.b_dtype = act, w.dtype, (bias.dtype if bias is not None else None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wf, bf = ctx.saved_tensors
        B, T, C = x.shape
        K = wf.shape[1]
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros_like(wf)
        db = torch.zeros(C, dtype=torch.float32, device=x.device) if bf is not None else None
        L.check(L.load().dewb_short_conv_bwd(L.ptr(x), L.ptr(dy), L.ptr(wf), L.ptr(bf), L.ptr(dx), L.ptr(dw), L.ptr(db),
                                             ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(C), ctypes.c_int(K),
                                             ctypes.c_int(int(ctx.act)), L.stream_ptr()), "short_conv_bwd")
        L.count_launches()
        return dx, dw.to(ctx.w_dtype), (db.to(ctx.b_dtype) if db is not None else None), None


def short_conv_cuda(x, w, bias=None, activation: bool = True):
    return _ShortConv.apply(x.contiguous(), w, bias, activation)
