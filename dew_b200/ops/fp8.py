"""fp8 (e4m3) row-wise-scaled products on the tcgen05 ``kind::f8f6f4`` path.

``A`` is quantised per row (token) and ``B`` per output channel, so ``D = diag(a_scale) (A_q B_q^T) diag(b_scale)`` is
exact in the scales and the tensor core accumulates the e4m3 products in fp32.  Used for the forward of dense and
expert (grouped) projections; gradients stay in bf16 (the usual recipe).  Capability: the reference's scaled fp8 GEMMs
(src/dew/nn/kernels/grouped_matmul.py ``MosaicStepScaledGmm`` :1725, ``MosaicMxGmm`` :1746; formats.py ``MxFp8`` :186).
Scaling granularity here is per row / per output channel rather than per 1x128 block.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch


def _grad_accumulates(p) -> bool:
    from .functional import grad_accumulates
    return grad_accumulates(p)

from . import library as L

c_ll, c_int = ctypes.c_longlong, ctypes.c_int
E4M3_MAX = 448.0


def quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [rows, d]`` -> (e4m3 values as ``float8_e4m3fn [rows, d]``, fp32 scales ``[rows]``)."""
    if L.use_cuda(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        x2 = x.contiguous()
        q = torch.empty(x2.shape, dtype=torch.float8_e4m3fn, device=x.device)
        s = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        L.check(L.load().dewb_quantize_rows_fp8(L.ptr(x2), L.ptr(q), L.ptr(s), c_ll(x2.shape[0]), c_int(x2.shape[1]), L.stream_ptr()),
                "quantize_rows_fp8")
        L.count_launches()
        return q, s
    amax = x.float().abs().amax(-1)
    s = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    return (x.float() / s[:, None]).to(torch.float8_e4m3fn), s


def gemm_fp8(aq, a_scale, bq, b_scale, tile_group: Optional[torch.Tensor] = None, groups: int = 1) -> torch.Tensor:
    """``[M, K] x [groups * N, K]^T -> [M, N]`` bf16.  With ``tile_group`` the rows of ``aq`` are expert-sorted and each
    128-row tile multiplies its own group's ``N`` rows of ``bq``."""
    M, K = aq.shape
    N = bq.shape[0] // groups
    if not L.use_cuda(aq):
        a = aq.float() * a_scale[:, None]
        b = bq.float() * b_scale[:, None]
        if tile_group is None:
            return (a @ b.t()).to(torch.bfloat16)
        out = torch.zeros(M, N)
        for t, g in enumerate(tile_group.tolist()):
            if g >= 0:
                out[t * 128:(t + 1) * 128] = a[t * 128:(t + 1) * 128] @ b[g * N:(g + 1) * N].t()
        return out.to(torch.bfloat16)
    out = torch.zeros((M, N), dtype=torch.bfloat16, device=aq.device) if tile_group is not None else \
        torch.empty((M, N), dtype=torch.bfloat16, device=aq.device)
    rc = L.load().dewb_gemm_fp8(L.ptr(aq), L.ptr(bq), L.ptr(out), L.ptr(a_scale), L.ptr(b_scale), L.ptr(tile_group), c_int(M), c_int(N),
                                c_int(K), c_int(groups), c_ll(aq.stride(0)), c_ll(bq.stride(0)), c_ll(out.stride(0)),
                                L.ptr(L.status(aq.device)), L.stream_ptr())
    L.check(rc, "gemm_fp8")
    L.count_launches()
    return out


class _Fp8GroupedLinear(torch.autograd.Function):
    """Forward in fp8 (activations quantised per token, weights per output channel); backward in bf16."""

    @staticmethod
    def forward(ctx, x, w, layout):
        from . import grouped as G
        ctx.layout = layout
        ctx.save_for_backward(x, w)
        G_, N, K = w.shape
        xq, xs = quantize_rows(x)
        wq, ws = quantize_rows(w.reshape(G_ * N, K))
        return gemm_fp8(xq, xs, wq, ws, layout.tile_group, G_)

    @staticmethod
    def backward(ctx, dy):
        from . import grouped as G
        x, w = ctx.saved_tensors
        layout = ctx.layout
        dy = dy.contiguous()
        dx = G.gmm_forward(dy, w, layout, transpose_w=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            if main is not None and dy.is_cuda:
                G.tgmm(dy, x, layout, w.shape[0], out=main, accumulate=_grad_accumulates(w))
            else:
                dw = G.tgmm(dy, x, layout, w.shape[0]).to(w.dtype)
        return dx, dw, None


def fp8_grouped_linear(x, w, layout):
    return _Fp8GroupedLinear.apply(x, w, layout)
