"""The op layer: every hot operation as one function with a CUDA path (sm_100a kernels from ``libdewb.so``)
and a PyTorch reference path that runs anywhere.

CUDA tensors always take the kernel path (missing library => loud failure).  CPU tensors take the reference
path, which is also the numerics oracle the GPU tests compare against.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import library as L
from .selection import Kernel, Requirement, op

c_ll = ctypes.c_longlong
c_int = ctypes.c_int
c_float = ctypes.c_float

# ---------------------------------------------------------------------------------------------------------------
# GEMM


def _gemm_reference(a, b, a_mn, b_mn, out_dtype, alpha, out, accumulate):
    A = a.t() if a_mn else a
    Bt = b if b_mn else b.t()
    r = (A.float() @ Bt.float()) * alpha
    if out is not None:
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r.to(out.dtype))
        return out
    return r.to(out_dtype)


_GEMM = op("gemm")
_GEMM.kernels = [
    Kernel("sm100_tcgen05", [
        Requirement("dtype", lambda c: c["dtype"] == torch.bfloat16, "operands must be bf16"),
        Requirement("ld", lambda c: c["lda"] % 8 == 0 and c["ldb"] % 8 == 0 and c["ldd"] % 8 == 0,
                    "row strides must be multiples of 8 elements (16-byte TMA rule)"),
        Requirement("align", lambda c: c["aligned"], "base pointers must be 16-byte aligned"),
        Requirement("inner", lambda c: c["inner_contig"], "the contiguous dimension must have stride 1"),
    ], receipt="tcgen05 128x256x64 persistent kernel, csrc/kernels/gemm_sm100.cu"),
    Kernel("sm100_pair", [
        Requirement("built", lambda c: _pair_built(), "the CTA-pair kernel is not in this build of libdewb.so"),
        Requirement("dtype", lambda c: c["dtype"] == torch.bfloat16, "operands must be bf16"),
        Requirement("ld", lambda c: c["lda"] % 8 == 0 and c["ldb"] % 8 == 0 and c["ldd"] % 8 == 0,
                    "row strides must be multiples of 8 elements (16-byte TMA rule)"),
        Requirement("align", lambda c: c["aligned"], "base pointers must be 16-byte aligned"),
        Requirement("inner", lambda c: c["inner_contig"], "the contiguous dimension must have stride 1"),
    ], receipt="tcgen05 cta_group::2 256x256x64 persistent kernel on CTA pairs, csrc/kernels/gemm_pair_sm100.cu"),
    Kernel("sm100_skinny", [
        Requirement("built", lambda c: _skinny_built(), "the weight-streaming kernel is not in this build of libdewb.so"),
        Requirement("rows", lambda c: c["M"] <= 128, "at most 128 rows (one tile of batch rows)"),
        Requirement("plain", lambda c: c.get("plain", False), "K-major operands, bf16 output, no accumulation, alpha = 1"),
        Requirement("dtype", lambda c: c["dtype"] == torch.bfloat16, "operands must be bf16"),
        Requirement("ld", lambda c: c["lda"] % 8 == 0 and c["ldb"] % 8 == 0 and c["K"] % 8 == 0,
                    "row strides and K must be multiples of 8 elements (16-byte TMA rule)"),
        Requirement("align", lambda c: c["aligned"], "base pointers must be 16-byte aligned"),
        Requirement("inner", lambda c: c["inner_contig"], "the contiguous dimension must have stride 1"),
    ], receipt="tcgen05 weight-streaming kernel, K split over a thread-block cluster and summed through distributed shared "
               "memory, csrc/kernels/gemm_skinny_sm100.cu"),
    Kernel("cublas", [], receipt="library arm (torch.matmul)"),
]


def _skinny_built() -> bool:
    try:
        return hasattr(L.load(), "dewb_gemm_skinny_bf16")
    except Exception:
        return False


def skinny_split(N: int, K: int, tile_cols: int = 128) -> int:
    """CTAs per output tile of the weight-streaming kernel: enough to cover the SMs, a power of two up to 8, and at least two
    reduction steps of 64 for every CTA."""
    tiles = -(-N // tile_cols)
    want = max(1, 148 // max(1, tiles))
    steps = -(-K // 64)
    split = 1
    while split * 2 <= min(8, want) and steps // (split * 2) >= 2:
        split *= 2
    return split


def _pair_built() -> bool:
    try:
        return hasattr(L.load(), "dewb_gemm_pair_bf16")
    except Exception:
        return False


_TUNE = bool(int(os.environ.get("DEWB_TUNE", "0")))
from .tuning import KernelOp as _KernelOp  # noqa: E402
_GEMM_TUNER = _KernelOp("gemm_bf16")

# Which of this library's two dense kernels large products take ("sm100_tcgen05" or "sm100_pair").
LARGE_GEMM = os.environ.get("DEWB_LARGE_GEMM", "sm100_pair")


# Measured cell: with fewer than ~24 output tiles of 128x256 (decode-sized products, e.g. 128 x 768) the persistent
# kernel leaves most SMs idle; the library's split-K kernels take those calls.
_GEMM.declared[("skinny",)] = "cublas"
# Decode-sized products (at most 128 rows) stream the weight once.  Measured inside the TP = 8 decode step: cuBLAS's small-tile kernels
# 6.6-7.6 us a call, this library's cluster split-K kernel 14.4 us - so the cell names the library arm; DEWB_DECODE_GEMM=sm100_skinny
# selects the weight-streaming kernel (and with it the SwiGLU epilogue of `linear_swiglu`).
_GEMM.declared[("decode",)] = os.environ.get("DEWB_DECODE_GEMM", "cublas")
_SKINNY_PDL = int(os.environ.get("DEWB_SKINNY_PDL", "1"))


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False,
         alpha: float = 1.0, max_ctas: int = 0, kernel: Optional[str] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``D[M,N] = alpha * op(a) @ op(b)^T (+ bias)`` with fp32 accumulation.  ``bias`` (one value per output column) is added in
    the epilogue of this library's dense kernels; the other routes add it afterwards.

    ``a`` is ``[M,K]`` (or stored ``[K,M]`` when ``a_mn``); ``b`` is ``[N,K]`` (or stored ``[K,N]`` when ``b_mn``).
    ``out`` (bf16 or fp32) may be given, and ``accumulate`` adds into it.
    """
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N = b.shape[1] if b_mn else b.shape[0]
    Kb = b.shape[0] if b_mn else b.shape[1]
    if K != Kb:
        raise ValueError(f"gemm: reduction sizes differ ({K} vs {Kb})")
    if not L.use_cuda(a, b):
        r = _gemm_reference(a, b, a_mn, b_mn, out_dtype, alpha, out, accumulate)
        return r if bias is None else r.add_(bias.to(r.dtype))
    if bias is not None and (accumulate or out is not None and out.dtype != torch.bfloat16 or out_dtype != torch.bfloat16):
        raise ValueError("gemm: a bias joins a fresh bf16 output only")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        accumulate = False
    case = dict(dtype=a.dtype if a.dtype == b.dtype else None, lda=a.stride(0), ldb=b.stride(0), ldd=out.stride(0),
                aligned=(a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0),
                inner_contig=(a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1), M=M, N=N, K=K,
                plain=(not a_mn and not b_mn and out.dtype == torch.bfloat16 and not accumulate and alpha == 1.0))
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    cell = ("decode",) if (M <= 128 and case["plain"] and bias is None) else (("skinny",) if tiles < 24 else None)
    if bias is not None:
        case["plain"] = False                                    # (the weight-streaming kernel has no bias epilogue)
    if kernel is None and cell is None and tiles >= 148 and _pair_built():
        # measured: the pair kernel is 5-15 % faster on the layer shapes; the single-CTA kernel keeps the very wide head.
        # With DEWB_TUNE=1 the two are timed once per shape and the pick is cached on disk (ops/tuning.py).
        first = "sm100_pair" if (LARGE_GEMM == "sm100_pair" and N <= 32768) else "sm100_tcgen05"
        other = "sm100_tcgen05" if first == "sm100_pair" else "sm100_pair"
        if _TUNE and not torch.cuda.is_current_stream_capturing():
            scratch = torch.empty_like(out)
            kernel = _GEMM_TUNER.pick((M, N, K, a_mn, b_mn, str(out.dtype), bool(accumulate)), [first, other],
                                      lambda name: gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=scratch, alpha=alpha, kernel=name), tune=True)
        else:
            kernel = first
    which = _GEMM.select(case, forced=kernel, cell=cell)
    if which == "cublas":
        r = _gemm_reference_cuda(a, b, a_mn, b_mn, alpha, out, accumulate)
        return r if bias is None else r.add_(bias.to(r.dtype))
    if which == "sm100_skinny":
        rc = L.load().dewb_gemm_skinny_bf16(L.ptr(a), L.ptr(b), L.ptr(out), c_int(M), c_int(N), c_int(K), c_ll(a.stride(0)), c_ll(b.stride(0)),
                                            c_ll(out.stride(0)), c_int(skinny_split(N, K)), c_int(0), c_int(_SKINNY_PDL),
                                            L.ptr(L.status(a.device)), L.stream_ptr())
        L.check(rc, which)
        L.count_launches()
        return out
    epi = {(torch.bfloat16, False): 0, (torch.float32, False): 1, (torch.float32, True): 2,
           (torch.bfloat16, True): 3}[(out.dtype, bool(accumulate))]
    lib = L.load()
    if bias is not None:
        bb = bias.to(torch.bfloat16).contiguous()                 # referenced until the launch is enqueued
        fn = lib.dewb_gemm_pair_bf16_bias if which == "sm100_pair" else lib.dewb_gemm_bf16_bias
        rc = fn(L.ptr(a), L.ptr(b), L.ptr(out), L.ptr(bb), c_int(M), c_int(N), c_int(K), c_ll(a.stride(0)),
                c_ll(b.stride(0)), c_ll(out.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)), c_int(epi),
                c_float(alpha), L.ptr(L.status(a.device)), c_int(max_ctas), L.stream_ptr())
        L.check(rc, which)
        L.count_launches()
        return out
    fn = lib.dewb_gemm_pair_bf16 if which == "sm100_pair" else lib.dewb_gemm_bf16
    rc = fn(L.ptr(a), L.ptr(b), L.ptr(out), c_int(M), c_int(N), c_int(K), c_ll(a.stride(0)),
            c_ll(b.stride(0)), c_ll(out.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)), c_int(epi),
            c_float(alpha), L.ptr(L.status(a.device)), c_int(max_ctas), L.stream_ptr())
    L.check(rc, which)
    L.count_launches()
    return out


def _gemm_reference_cuda(a, b, a_mn, b_mn, alpha, out, accumulate):
    A = a.t() if a_mn else a
    Bt = b if b_mn else b.t()
    if out.dtype == a.dtype and not accumulate and alpha == 1.0:
        torch.matmul(A, Bt, out=out)
    else:
        r = torch.matmul(A, Bt)
        if accumulate:
            out.add_(r, alpha=alpha)
        else:
            out.copy_(r if alpha == 1.0 else r * alpha)
    return out


def grad_accumulates(p) -> bool:
    """Whether a weight gradient written into ``p.main_grad`` adds to what is there.  An engine that reuses one gradient
    buffer for several units marks a parameter's buffer as stale (``p._dewb_fresh = True``); the first write after that
    overwrites instead of accumulating, and clears the mark."""
    if getattr(p, "_dewb_fresh", False):
        p._dewb_fresh = False
        return False
    return True


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, weight, bias=bias)                          # the bias joins in the product's epilogue
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).reshape(x.shape)            # dY[M,N] @ W[N,K]
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "main_grad", None)
            if main is not None:                                           # fused accumulation into the fp32 buffer
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=grad_accumulates(weight))
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)                   # dY^T[N,M] @ x[M,K]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = x @ weight^T + bias`` with ``weight`` stored ``[out, in]``."""
    if not L.use_cuda(x, weight) or x.dtype != torch.bfloat16:
        return F.linear(x, weight.to(x.dtype) if weight.dtype != x.dtype else weight, bias)
    if not x.is_contiguous():
        x = x.contiguous()
    return _Linear.apply(x, weight, bias)


# ---------------------------------------------------------------------------------------------------------------
# RMSNorm family


def rms_norm_reference(x, w, eps=1e-6):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


class _L2Norm(torch.autograd.Function):
    """``y = x / max(||x||, eps)`` over the last axis on the row kernel (``csrc/kernels/l2norm.cu``); x may be a strided
    ``[B, T, H, D]`` view of a wider projection, y and dx are contiguous."""

    @staticmethod
    def forward(ctx, x, eps):
        B, T, H, D = x.shape
        rows = B * T * H
        y = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=x.device)
        rnorm = torch.empty(rows, dtype=torch.float32, device=x.device)
        L.ensure_device(x)
        L.check(L.load().dewb_l2norm_fwd(L.ptr(x), L.ptr(y), L.ptr(rnorm), ctypes.c_longlong(rows), ctypes.c_int(H),
                                         ctypes.c_longlong(x.stride(1)), ctypes.c_longlong(x.stride(2)), ctypes.c_int(D),
                                         ctypes.c_float(eps), L.stream_ptr()), "l2norm_fwd")
        L.count_launches()
        ctx.save_for_backward(y, rnorm)
        return y

    @staticmethod
    def backward(ctx, dy):
        y, rnorm = ctx.saved_tensors
        dy = dy.contiguous().to(torch.bfloat16)
        dx = torch.empty_like(y)
        L.ensure_device(y)
        L.check(L.load().dewb_l2norm_bwd(L.ptr(y), L.ptr(dy), L.ptr(rnorm), L.ptr(dx), ctypes.c_longlong(rnorm.numel()),
                                         ctypes.c_int(y.shape[-1]), L.stream_ptr()), "l2norm_bwd")
        L.count_launches()
        return dx, None


def l2_normalize(x: torch.Tensor, eps: float = 1e-12) -> torch.Tensor:
    """``x [B, T, H, D] -> x / max(||x||_2, eps)`` over D.  bf16 CUDA tensors (D <= 1024, D % 8 == 0) run the row kernel and
    return bf16; anything else is ``F.normalize`` in fp32."""
    if (x.dim() == 4 and x.dtype == torch.bfloat16 and L.use_cuda(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 1024
            and hasattr(L.load(), "dewb_l2norm_fwd")):
        if not (x.stride(3) == 1 and x.stride(0) == x.shape[1] * x.stride(1) and x.stride(1) % 8 == 0 and x.stride(2) % 8 == 0
                and x.data_ptr() % 16 == 0):
            x = x.contiguous()
        return _L2Norm.apply(x, float(eps))
    return torch.nn.functional.normalize(x.float(), dim=-1, eps=eps)


def _bwd_scratch(rows: int, d: int, device) -> torch.Tensor:
    blocks = L.load().dewb_rmsnorm_bwd_blocks(c_ll(rows))
    return torch.empty((blocks, d), dtype=torch.float32, device=device)


class _RMSNorm(torch.autograd.Function):
    """mode 0 plain, 1 stream (x + branch, emits both), 2 gated (norm(x) * w * silu(z))."""

    @staticmethod
    def forward(ctx, x, other, w, eps, mode):
        lib = L.load()
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        rows = x2.shape[0]
        o2 = other.reshape(-1, d) if other is not None else None
        y = torch.empty_like(x2)
        h = torch.empty_like(x2) if mode == 1 else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        wb = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        L.check(lib.dewb_rmsnorm_fwd(L.ptr(x2), L.ptr(o2), L.ptr(wb), L.ptr(y), L.ptr(h), L.ptr(rstd), c_ll(rows),
                                     c_int(d), c_float(eps), c_int(mode), L.stream_ptr()), "rmsnorm_fwd")
        L.count_launches()
        ctx.mode, ctx.shape = mode, x.shape
        ctx.save_for_backward(h if mode == 1 else x2, wb, rstd, o2 if mode == 2 else None)
        ctx.w_dtype = w.dtype
        if mode == 1:
            ctx.mark_non_differentiable()
            return y.reshape(x.shape), h.reshape(x.shape)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        xin, wb, rstd, z = ctx.saved_tensors
        lib = L.load()
        d = xin.shape[-1]
        rows = xin.shape[0]
        dy2 = dy.reshape(-1, d).contiguous()
        dres = dh.reshape(-1, d).contiguous() if (ctx.mode == 1 and dh is not None) else None
        dx = torch.empty_like(xin)
        dz = torch.empty_like(xin) if ctx.mode == 2 else None
        dw = torch.empty(d, dtype=torch.float32, device=xin.device)
        scratch = _bwd_scratch(rows, d, xin.device)
        L.check(lib.dewb_rmsnorm_bwd(L.ptr(dy2), L.ptr(xin), L.ptr(wb), L.ptr(rstd), L.ptr(dres), L.ptr(z), L.ptr(dx),
                                     L.ptr(dz), L.ptr(scratch), L.ptr(dw), L.ptr(None), c_int(0), c_ll(rows), c_int(d),
                                     L.stream_ptr()), "rmsnorm_bwd")
        L.count_launches(2)
        dxr = dx.reshape(ctx.shape)
        dwr = dw.to(ctx.w_dtype)
        if ctx.mode == 1:
            return dxr, dxr, dwr, None, None
        if ctx.mode == 2:
            return dxr, dz.reshape(ctx.shape), dwr, None, None
        return dxr, None, dwr, None, None


def _norm_cuda_ok(x, w):
    return x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if L.use_cuda(x) and _norm_cuda_ok(x, w):
        return _RMSNorm.apply(x.contiguous(), None, w, eps, 0)
    return rms_norm_reference(x, w, eps)


def stream_rms_norm(x: torch.Tensor, branch: torch.Tensor, w: torch.Tensor, eps: float = 1e-6):
    """Residual-stream norm: ``h = x + branch``; returns ``(norm(h) * w, h)`` from one pass."""
    if L.use_cuda(x) and _norm_cuda_ok(x, w):
        return _RMSNorm.apply(x.contiguous(), branch.contiguous(), w, eps, 1)
    h = (x.float() + branch.float()).to(x.dtype)
    return rms_norm_reference(h, w, eps), h


def gated_rms_norm(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``norm(x) * w * silu(z)`` (the output gate of gated-delta-net / Mamba-2 blocks)."""
    if L.use_cuda(x) and _norm_cuda_ok(x, w):
        return _RMSNorm.apply(x.contiguous(), z.contiguous(), w, eps, 2)
    return (rms_norm_reference(x, w, eps).float() * F.silu(z.float())).to(x.dtype)


# ---------------------------------------------------------------------------------------------------------------
# SwiGLU


class _PackedSwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        lib = L.load()
        F2 = gu.shape[-1]
        Fh = F2 // 2
        g2 = gu.reshape(-1, F2)
        rows = g2.shape[0]
        out = torch.empty((rows, Fh), dtype=gu.dtype, device=gu.device)
        L.check(lib.dewb_swiglu_fwd(L.ptr(g2), ctypes.c_void_p(g2.data_ptr() + Fh * 2), L.ptr(out), c_ll(rows),
                                    c_int(Fh), c_ll(F2), L.stream_ptr()), "swiglu_fwd")
        L.count_launches()
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.reshape(*gu.shape[:-1], Fh)

    @staticmethod
    def backward(ctx, dy):
        (g2,) = ctx.saved_tensors
        lib = L.load()
        F2 = g2.shape[-1]
        Fh = F2 // 2
        rows = g2.shape[0]
        dy2 = dy.reshape(-1, Fh).contiguous()
        dgu = torch.empty_like(g2)
        L.check(lib.dewb_swiglu_bwd(L.ptr(dy2), L.ptr(g2), ctypes.c_void_p(g2.data_ptr() + Fh * 2), L.ptr(dgu),
                                    ctypes.c_void_p(dgu.data_ptr() + Fh * 2), c_ll(rows), c_int(Fh), c_ll(F2),
                                    L.stream_ptr()), "swiglu_bwd")
        L.count_launches()
        return dgu.reshape(ctx.shape)


def packed_swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gu[..., :F]) * gu[..., F:]`` on the output of a fused gate|up projection."""
    Fh = gu.shape[-1] // 2
    if L.use_cuda(gu) and gu.dtype == torch.bfloat16 and Fh % 8 == 0:
        return _PackedSwiGLU.apply(gu.contiguous())
    g, u = gu[..., :Fh], gu[..., Fh:]
    return (F.silu(g.float()) * u.float()).to(gu.dtype)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, fused: Optional[bool] = None) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)`` for the packed ``[2 F, d]`` weight.  Decode-sized inputs (at most 128 rows, no autograd) run as ONE
    kernel when the weight-streaming GEMM is the decode cell's choice (or ``fused=True``): it applies the activation in its epilogue, so
    the ``[rows, 2 F]`` intermediate never exists."""
    Fh = w_gate_up.shape[0] // 2
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    if (L.use_cuda(x2, w_gate_up) and M <= 128 and x2.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and Fh % 64 == 0
            and K % 8 == 0 and x2.stride(1) == 1 and x2.stride(0) % 8 == 0 and w_gate_up.is_contiguous() and x2.data_ptr() % 16 == 0
            and not (torch.is_grad_enabled() and (x.requires_grad or w_gate_up.requires_grad)) and _skinny_built()
            and (fused if fused is not None else _GEMM.declared.get(("decode",)) == "sm100_skinny")):
        out = torch.empty((M, Fh), dtype=torch.bfloat16, device=x.device)
        rc = L.load().dewb_gemm_skinny_bf16(L.ptr(x2), L.ptr(w_gate_up), L.ptr(out), c_int(M), c_int(Fh), c_int(K), c_ll(x2.stride(0)),
                                            c_ll(w_gate_up.stride(0)), c_ll(Fh), c_int(skinny_split(Fh, K, 64)), c_int(1), c_int(_SKINNY_PDL),
                                            L.ptr(L.status(x.device)), L.stream_ptr())
        L.check(rc, "sm100_skinny")
        L.count_launches()
        return out.reshape(*x.shape[:-1], Fh)
    return packed_swiglu(linear(x, w_gate_up))


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return packed_swiglu(torch.cat([gate, up], -1)) if gate.is_cuda else (F.silu(gate.float()) * up.float()).to(gate.dtype)


# ---------------------------------------------------------------------------------------------------------------
# RoPE


def rope_tables(max_pos: int, dim: int, theta: float = 10000.0, device="cpu", scaling: Optional[dict] = None, rotary_dim: Optional[int] = None):
    """cos/sin tables ``[max_pos, dim/2]`` in fp32 (rotate-half convention).  ``rotary_dim < dim`` (partial rotary): the frequencies are
    those of a ``rotary_dim``-wide rotation and fill the first ``rotary_dim / 2`` columns; the others hold the identity (cos 1, sin 0),
    so a head laid out ``[rotated a | kept a | rotated b | kept b]`` passes its kept dimensions through the same kernel unchanged.  ``scaling`` (keyed by ``type`` or ``rope_type``):
    ``linear`` (``factor``); ``llama3`` (``factor, low_freq_factor, high_freq_factor, original_max_position_embeddings``);
    ``yarn`` (``factor, original_max_position_embeddings, beta_fast, beta_slow, mscale, mscale_all_dim, attention_factor, truncate``:
    high frequencies extrapolate, low ones interpolate, a ramp between, and the tables carry the attention factor);
    ``longrope`` (``short_factor`` / ``long_factor`` per frequency: the long set when the table is longer than
    ``original_max_position_embeddings``, else the short one); ``dynamic`` (NTK-aware: the base grows with the table's length over the original
    context).  A kind this function does not know raises: silently unscaled positions
    would read as a model that has forgotten its long context."""
    full = dim
    if rotary_dim is not None and rotary_dim < dim:
        if rotary_dim % 2 or (dim - rotary_dim) % 2:
            raise ValueError(f"partial rotary wants even widths, got {rotary_dim} of {dim}")
        dim = rotary_dim
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64, device=device) / dim))
    amplitude = 1.0
    if scaling:
        kind = scaling.get("type", scaling.get("rope_type", "linear"))
        if kind == "default":
            pass
        elif kind == "linear":
            inv = inv / scaling["factor"]
        elif kind == "llama3":
            f, lo, hi = scaling["factor"], scaling.get("low_freq_factor", 1.0), scaling.get("high_freq_factor", 4.0)
            orig = scaling.get("original_max_position_embeddings", 8192)
            wavelen = 2 * math.pi / inv
            smooth = ((orig / wavelen) - lo) / (hi - lo)
            scaled = torch.where(wavelen > orig / lo, inv / f, inv)
            mid = (wavelen <= orig / lo) & (wavelen >= orig / hi)
            inv = torch.where(mid, (1 - smooth) * inv / f + smooth * inv, scaled)
        elif kind == "yarn":
            orig = scaling.get("original_max_position_embeddings") or max_pos
            f = scaling.get("factor") or max_pos / orig

            def magnitude(s, m=1.0):
                return 1.0 if s <= 1 else 0.1 * m * math.log(s) + 1.0
            amplitude = scaling.get("attention_factor")
            if amplitude is None:
                m, m_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
                amplitude = magnitude(f, m) / magnitude(f, m_all) if m and m_all else magnitude(f)

            def turns_to_index(n):               # the frequency index whose wave makes n turns over the original context
                return dim * math.log(orig / (n * 2 * math.pi)) / (2 * math.log(theta))
            lo, hi = turns_to_index(scaling.get("beta_fast") or 32), turns_to_index(scaling.get("beta_slow") or 1)
            if scaling.get("truncate", True):
                lo, hi = math.floor(lo), math.ceil(hi)
            lo, hi = max(lo, 0), min(hi, dim - 1)
            if lo == hi:
                hi += 0.001
            keep = 1.0 - ((torch.arange(dim // 2, dtype=torch.float64, device=device) - lo) / (hi - lo)).clamp(0, 1)
            inv = inv / f * (1 - keep) + inv * keep
        elif kind == "longrope":
            orig = scaling.get("original_max_position_embeddings") or max_pos
            which = "long_factor" if max_pos > orig else "short_factor"
            inv = inv / torch.tensor(scaling[which], dtype=torch.float64, device=device)
            f = scaling.get("factor") or max_pos / orig
            amplitude = scaling.get("attention_factor")
            if amplitude is None:
                amplitude = 1.0 if f <= 1 else math.sqrt(1 + math.log(f) / math.log(orig))
        elif kind == "dynamic":
            # NTK-aware scaling by the length in use; a table is built once for max_pos positions, so that is the length it is scaled for
            orig = scaling.get("original_max_position_embeddings") or max_pos
            if max_pos > orig:
                base = theta * ((scaling["factor"] * max_pos / orig) - (scaling["factor"] - 1)) ** (dim / (dim - 2))
                inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float64, device=device) / dim))
        else:
            raise ValueError(f"rotary scaling {kind!r} is not built (known: linear, llama3, yarn, longrope, dynamic)")
    t = torch.arange(max_pos, dtype=torch.float64, device=device)
    ang = torch.outer(t, inv)
    cos, sin = ang.cos() * amplitude, ang.sin() * amplitude
    if full != dim:
        cos = torch.cat([cos, torch.ones(max_pos, (full - dim) // 2, dtype=cos.dtype, device=cos.device)], 1)
        sin = torch.cat([sin, torch.zeros(max_pos, (full - dim) // 2, dtype=sin.dtype, device=sin.device)], 1)
    return cos.float().contiguous(), sin.float().contiguous()


def rope_reference(x, cos, sin, positions=None, rot_heads=None):
    """x [..., T, H, D]; cos/sin [P, D/2]."""
    T, H, D = x.shape[-3], x.shape[-2], x.shape[-1]
    if positions is None:
        c, s = cos[:T], sin[:T]
    else:
        c, s = cos[positions.long()], sin[positions.long()]
    c = c.reshape(*([1] * (x.dim() - 3)), *c.shape[:-1], 1, D // 2) if positions is None else c.unsqueeze(-2)
    s = s.reshape(*([1] * (x.dim() - 3)), *s.shape[:-1], 1, D // 2) if positions is None else s.unsqueeze(-2)
    xf = x.float()
    x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    if rot_heads is not None and rot_heads < H:
        out = torch.cat([out[..., :rot_heads, :], xf[..., rot_heads:, :]], -2)
    return out.to(x.dtype)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, positions, rot_heads):
        lib = L.load()
        H, D = x.shape[-2], x.shape[-1]
        out = x.clone()
        tokens = out.numel() // (H * D)
        pos = None
        if positions is not None:
            pos = positions.reshape(-1).to(torch.int32).contiguous()
        elif out.dim() == 4 and out.shape[0] > 1:
            pos = torch.arange(out.shape[1], device=x.device, dtype=torch.int32).repeat(out.shape[0])
        L.check(lib.dewb_rope(L.ptr(out), L.ptr(cos), L.ptr(sin), L.ptr(pos), c_ll(tokens), c_int(H), c_int(rot_heads),
                              c_int(D), c_int(cos.shape[0]), c_float(1.0), L.stream_ptr()), "rope")
        L.count_launches()
        ctx.save_for_backward(cos, sin, pos)
        ctx.rot_heads = rot_heads
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pos = ctx.saved_tensors
        lib = L.load()
        H, D = dy.shape[-2], dy.shape[-1]
        dx = dy.clone() if not dy.is_contiguous() else dy.clone()
        dx = dx.contiguous()
        tokens = dx.numel() // (H * D)
        L.check(lib.dewb_rope(L.ptr(dx), L.ptr(cos), L.ptr(sin), L.ptr(pos), c_ll(tokens), c_int(H),
                              c_int(ctx.rot_heads), c_int(D), c_int(cos.shape[0]), c_float(-1.0), L.stream_ptr()), "rope_bwd")
        L.count_launches()
        return dx, None, None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: Optional[torch.Tensor] = None,
         rot_heads: Optional[int] = None) -> torch.Tensor:
    """Rotate the first ``rot_heads`` heads of ``x [B, T, H, D]`` (all by default)."""
    H, D = x.shape[-2], x.shape[-1]
    rh = H if rot_heads is None else rot_heads
    if L.use_cuda(x) and x.dtype == torch.bfloat16 and D % 16 == 0:
        return _Rope.apply(x.contiguous(), cos, sin, positions, rh)
    return rope_reference(x, cos.to(x.device), sin.to(x.device), positions, rh)


# ---------------------------------------------------------------------------------------------------------------
# Attention


def attention_reference(q, k, v, causal=True, scale=None, window=None, softcap=0.0, sinks=None, segment_ids=None):
    """q [B,S,Hq,D], k/v [B,T,Hkv,D] -> [B,S,Hq,D]; fp32 math; GQA by head repetition."""
    B, S, Hq, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if softcap and softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    qi = torch.arange(S, device=q.device)[:, None] + (T - S)
    ki = torch.arange(T, device=q.device)[None, :]
    mask = torch.ones(S, T, dtype=torch.bool, device=q.device)
    if causal:
        mask &= ki <= qi
    if window is not None:
        mask &= ki > qi - window
    mask = mask[None, None]
    if segment_ids is not None:
        seg = segment_ids
        mask = mask & (seg[:, None, -S:, None] == seg[:, None, None, :])
    s = s.masked_fill(~mask, float("-inf"))
    if sinks is not None:
        sink = sinks.float().reshape(1, Hq, 1, 1).expand(B, Hq, S, 1)
        p = torch.softmax(torch.cat([s, sink], -1), -1)[..., :-1]
    else:
        p = torch.softmax(s, -1)
    p = torch.nan_to_num(p)
    return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)


def attention(q, k, v, causal: bool = True, scale: Optional[float] = None, window: Optional[int] = None,
              softcap: float = 0.0, sinks=None, segment_ids=None, kernel: Optional[str] = None):
    """Scaled-dot-product attention with GQA; layouts ``[B, S, H, D]``."""
    if L.use_cuda(q):
        from . import attn as A
        return A.flash_attention(q, k, v, causal=causal, scale=scale, window=window, softcap=softcap, sinks=sinks,
                                 segment_ids=segment_ids, kernel=kernel)
    return attention_reference(q, k, v, causal, scale, window, softcap, sinks, segment_ids)


# ---------------------------------------------------------------------------------------------------------------
# Fused linear + cross-entropy head (never materialises [T, V] for the whole batch)


def linear_cross_entropy_reference(h, weight, targets, ignore_index=-100, z_loss=0.0, softcap=0.0):
    logits = h.float() @ weight.float().t()
    if softcap and softcap > 0:
        logits = softcap * torch.tanh(logits / softcap)
    lse = torch.logsumexp(logits, -1)
    live = targets != ignore_index
    tl = logits.gather(-1, targets.clamp_min(0).unsqueeze(-1)).squeeze(-1)
    loss = (lse - tl + z_loss * lse * lse) * live
    return loss.sum(), live.sum()


class _LinearCE(torch.autograd.Function):
    """Token-chunked head: per chunk, logits = h W^T (tcgen05 GEMM), a row kernel reduces the loss and overwrites
    the logits with their gradient, and two more GEMMs produce dH and accumulate dW - all inside forward, so the
    backward only rescales (the Liger construction; reference: src/dew/objectives/lm/chunked.py:774-874 tiles the
    same computation over tokens x vocabulary)."""

    @staticmethod
    def forward(ctx, h, weight, targets, ignore_index, z_loss, softcap, chunk):
        lib = L.load()
        T, d = h.shape
        V = weight.shape[0]
        need_grad = h.requires_grad or weight.requires_grad
        dh = torch.empty_like(h) if need_grad else None
        main = getattr(weight, "main_grad", None)
        dw = None
        if need_grad and weight.requires_grad and main is None:
            dw = torch.zeros((V, d), dtype=torch.float32, device=h.device)
        acc = main if main is not None else dw
        losses = torch.empty(T, dtype=torch.float32, device=h.device)
        tg = targets.to(torch.int64).contiguous()
        logits = torch.empty((min(chunk, T), V), dtype=torch.bfloat16, device=h.device)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            n = e - s
            lg = logits[:n]
            gemm(h[s:e], weight, out=lg)
            L.check(lib.dewb_ce_rows(L.ptr(lg), ctypes.c_void_p(tg.data_ptr() + s * 8),
                                     ctypes.c_void_p(losses.data_ptr() + s * 4), L.ptr(None), c_ll(n), c_int(V),
                                     c_ll(lg.stride(0)), c_int(ignore_index), c_float(1.0), c_float(z_loss),
                                     c_float(softcap), c_int(int(need_grad)), L.stream_ptr()), "ce_rows")
            L.count_launches()
            if need_grad:
                gemm(lg, weight, b_mn=True, out=dh[s:e])                       # dH = dlogits @ W
                if acc is not None:
                    gemm(lg, h[s:e], a_mn=True, b_mn=True, out=acc,
                         accumulate=grad_accumulates(weight) if main is not None else True)    # dW += dlogits^T @ h
        ctx.save_for_backward(dh, dw)
        ctx.used_main = main is not None
        ctx.w_dtype = weight.dtype
        live = (tg != ignore_index).sum()
        return losses.sum(), live

    @staticmethod
    def backward(ctx, gloss, glive):
        dh, dw = ctx.saved_tensors
        gh = (dh * gloss.to(dh.dtype)) if dh is not None else None
        gw = None
        if dw is not None:
            gw = (dw * gloss).to(ctx.w_dtype)
        return gh, gw, None, None, None, None, None


def linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100,
                         z_loss: float = 0.0, softcap: float = 0.0, chunk: int = 4096):
    """Summed token loss and live-token count of ``softmax(h @ weight^T)`` against ``targets``.

    ``h [T, d]``, ``weight [V, d]``, ``targets [T]``.  Returns ``(sum of losses, number of scored tokens)`` - a
    ``Ratio(total, mass)`` pair; divide once after pooling across microbatches and ranks.
    When ``weight.main_grad`` exists, dW is accumulated there in fp32 (pre-scaled by 1: callers that use
    ``main_grad`` must backpropagate a unit gradient into the summed loss).
    """
    if L.use_cuda(h) and h.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and h.shape[1] % 8 == 0:
        ctile = int(os.environ.get("DEWB_CE_CHUNK", chunk))
        return _LinearCE.apply(h.contiguous(), weight, targets, ignore_index, z_loss, softcap, ctile)
    T = h.shape[0]
    total = h.new_zeros((), dtype=torch.float32)
    mass = torch.zeros((), dtype=torch.long, device=h.device)
    for s in range(0, T, chunk):
        t, m = linear_cross_entropy_reference(h[s:s + chunk], weight, targets[s:s + chunk], ignore_index, z_loss, softcap)
        total = total + t
        mass = mass + m
    return total, mass


# ---------------------------------------------------------------------------------------------------------------
# Optimizer kernels on flat buffers


def grad_norm_(grads: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, max_norm: float = 0.0,
               accumulate: bool = False) -> torch.Tensor:
    """``out[0:3] = (sum of squares, norm, clip coefficient)`` of a flat gradient buffer, on device."""
    if L.use_cuda(grads):
        lib = L.load()
        L.check(lib.dewb_grad_norm(L.ptr(grads), c_ll(grads.numel()), c_int(int(grads.dtype == torch.bfloat16)),
                                   L.ptr(scratch), L.ptr(out), c_float(max_norm), c_int(int(accumulate)),
                                   L.stream_ptr()), "grad_norm")
        L.count_launches(2)
        return out
    ss = grads.float().pow(2).sum() + (out[0] if accumulate else 0.0)
    norm = ss.sqrt()
    out[0], out[1] = ss, norm
    out[2] = torch.where((norm > max_norm) & (max_norm > 0), max_norm / (norm + 1e-6), torch.ones_like(norm))
    return out


def adamw_(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, *, step: int, lr: float,
           beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0,
           p_bf16: Optional[torch.Tensor] = None, ema: Optional[torch.Tensor] = None, ema_decay: float = 0.0,
           grad_scale: float = 1.0, clip: Optional[torch.Tensor] = None, skip_nonfinite: bool = False) -> None:
    """In-place AdamW on flat fp32 ``p, m, v`` with gradient ``g`` (bf16 or fp32); refreshes the bf16 compute copy
    and the EMA in the same pass (reference semantics: src/dew/optim.py:1114 AdamW, src/dew/averaging.py:116-139)."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if L.use_cuda(p):
        lib = L.load()
        L.check(lib.dewb_adamw(L.ptr(p), L.ptr(m), L.ptr(v), L.ptr(g), c_int(int(g.dtype == torch.bfloat16)),
                               L.ptr(p_bf16), L.ptr(ema), c_ll(p.numel()), c_float(lr), c_float(beta1), c_float(beta2),
                               c_float(eps), c_float(weight_decay), c_float(bc1), c_float(bc2), c_float(grad_scale),
                               L.ptr(clip), c_float(ema_decay), c_int(int(skip_nonfinite)), L.stream_ptr()), "adamw")
        L.count_launches()
        return
    coef = grad_scale
    if clip is not None:
        if skip_nonfinite and not bool(torch.isfinite(clip[0])):
            return
        coef = coef * float(clip[2])
    gf = g.float() * coef
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    p.mul_(1 - lr * weight_decay).addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
    if p_bf16 is not None:
        p_bf16.copy_(p)
    if ema is not None:
        ema.mul_(ema_decay).add_(p, alpha=1 - ema_decay)


def ema_(ema: torch.Tensor, live: torch.Tensor, decay: float) -> None:
    if L.use_cuda(ema) and ema.dtype == torch.float32 and live.dtype == torch.float32:
        L.check(L.load().dewb_ema(L.ptr(ema), L.ptr(live), c_ll(ema.numel()), c_float(decay), L.stream_ptr()), "ema")
        L.count_launches()
        return
    ema.mul_(decay).add_(live.to(ema.dtype), alpha=1 - decay)
