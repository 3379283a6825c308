"""MXFP8 block-scaled products: e4m3 values with one power-of-two (ue8m0) scale per 32 consecutive elements of the
reduction dimension, multiplied by ``tcgen05.mma kind::mxf8f6f4.block_scale`` (``csrc/kernels/gemm_mx_sm100.cu``).

``quantize_mx``       ``x [rows, K]`` -> e4m3 values, packed scales (one 32-bit word per row per 128 elements)
``gemm_mx``           ``A_q [M, K] x B_q [G * N, K]^T`` -> ``[M, N]`` bf16, dense or grouped by 128-row tiles (experts)
``mx_grouped_linear`` differentiable expert projection: forward and input gradient in MXFP8 (the input gradient reduces over
                      the output features, so it uses the weights re-quantised along that dimension), weight gradient in bf16

On CPU the same arithmetic runs in PyTorch (quantise, de-quantise, fp32 product): the oracle of the kernel tests.
Reference: ``MxFp8`` 1 x 32 blocks with e8m0 scales (src/dew/nn/kernels/formats.py:186), ``MosaicMxGmm``
(src/dew/nn/kernels/grouped_matmul.py:1746).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import library as L

c_ll, c_int = ctypes.c_longlong, ctypes.c_int
BLOCK = 32
E4M3_MAX = 448.0
TILE_N = 192


def _pad128(n: int) -> int:
    return (n + 127) // 128 * 128


def quantize_mx_reference(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [rows, K]`` -> (``float8_e4m3fn [rows, K]``, exponents ``int32 [rows, K / 32]``: the block's scale is ``2 ** e``)."""
    rows, K = x.shape
    xb = x.float().reshape(rows, K // BLOCK, BLOCK)
    amax = xb.abs().amax(-1)
    # smallest integer e with amax <= 448 * 2^e, exactly: amax = m * 2^ex with m in [0.5, 1) and 448 = 0.875 * 2^9
    m, ex = torch.frexp(torch.where(amax > 0, amax, torch.ones_like(amax)))
    e = (ex - 9 + (m > 0.875).to(ex.dtype)).float()
    e = torch.where(amax > 0, e, torch.full_like(e, -127.0)).clamp(-127, 127)
    q = (xb * torch.exp2(-e)[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).reshape(rows, K)
    return q, e.to(torch.int32)


def dequantize_mx(q: torch.Tensor, e: torch.Tensor) -> torch.Tensor:
    rows, K = q.shape
    return (q.float().reshape(rows, K // BLOCK, BLOCK) * torch.exp2(e.float())[..., None]).reshape(rows, K)


def unpack_scales(sf: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """Packed scale words ``[K / 128, sf_rows]`` -> exponents ``int32 [rows, K / 32]``."""
    b = sf.view(torch.uint8).reshape(sf.shape[0], sf.shape[1], 4)[:, :rows]          # [kb, rows, 4]
    return (b.permute(1, 0, 2).reshape(rows, -1)[:, : K // BLOCK].to(torch.int32) - 127)


def quantize_mx(x: torch.Tensor, sf_rows: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [rows, K]`` bf16 (K a multiple of 128) -> (e4m3 ``[rows, K]``, packed scales ``int32 [K / 128, sf_rows]``)."""
    rows, K = x.shape
    if K % 128:
        raise ValueError(f"MXFP8 products need a reduction size that is a multiple of 128, got {K}")
    sf_rows = sf_rows if sf_rows is not None else _pad128(rows)
    if L.use_cuda(x) and x.dtype == torch.bfloat16:
        x2 = x if x.stride(1) == 1 else x.contiguous()
        q = torch.empty((rows, K), dtype=torch.float8_e4m3fn, device=x.device)
        sf = torch.zeros((K // 128, sf_rows), dtype=torch.int32, device=x.device)
        L.check(L.load().dewb_quantize_mx(L.ptr(x2), L.ptr(q), L.ptr(sf), c_ll(rows), c_int(K), c_ll(x2.stride(0)), c_ll(sf_rows),
                                          L.stream_ptr()), "quantize_mx")
        L.count_launches()
        return q, sf
    q, e = quantize_mx_reference(x)
    packed = torch.zeros((K // 128, sf_rows, 4), dtype=torch.uint8, device=x.device)
    packed[:, :rows] = (e + 127).to(torch.uint8).reshape(rows, K // 128, 4).permute(1, 0, 2)
    return q, packed.view(torch.int32).reshape(K // 128, sf_rows)


def gemm_mx(aq, sfa, bq, sfb, tile_group: Optional[torch.Tensor] = None, groups: int = 1, out: Optional[torch.Tensor] = None,
            zero_skipped: bool = True) -> torch.Tensor:
    """``[M, K] x [groups * N, K]^T -> [M, N]`` bf16.  With ``tile_group`` the rows of ``aq`` are expert-sorted and each 128-row
    tile multiplies its own group's ``N`` rows of ``bq``.  ``sfb`` must have at least ``groups * N + 192`` rows.  ``out``: write
    into this ``[M, N]`` bf16 tensor.  Row tiles without a group are not written: with ``zero_skipped`` (default) they read zero,
    without it they keep whatever the memory held - enough when nothing downstream reads them (an expert pipeline whose every
    consumer walks the same tiles)."""
    M, K = aq.shape
    N = bq.shape[0] // groups
    if not L.use_cuda(aq):
        a = dequantize_mx(aq, unpack_scales(sfa, M, K))
        b = dequantize_mx(bq, unpack_scales(sfb, bq.shape[0], K))
        if tile_group is None:
            res = (a @ b.t()).to(torch.bfloat16)
        else:
            res = torch.zeros(M, N)
            for t, g in enumerate(tile_group.tolist()):
                if g >= 0:
                    res[t * 128:(t + 1) * 128] = a[t * 128:(t + 1) * 128] @ b[g * N:(g + 1) * N].t()
            res = res.to(torch.bfloat16)
        return res if out is None else out.copy_(res)
    if out is None:
        out = torch.zeros((M, N), dtype=torch.bfloat16, device=aq.device) if (tile_group is not None and zero_skipped) else \
            torch.empty((M, N), dtype=torch.bfloat16, device=aq.device)
    elif tuple(out.shape) != (M, N) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("gemm_mx: `out` must be a contiguous [M, N] bf16 tensor")
    elif tile_group is not None and zero_skipped:
        out.zero_()
    rc = L.load().dewb_gemm_mxfp8(L.ptr(aq), L.ptr(bq), L.ptr(out), L.ptr(sfa), L.ptr(sfb), L.ptr(tile_group), c_int(M), c_int(N),
                                  c_int(K), c_int(groups), c_ll(aq.stride(0)), c_ll(bq.stride(0)), c_ll(out.stride(0)),
                                  c_ll(sfa.shape[1]), c_ll(sfb.shape[1]), L.ptr(L.status(aq.device)), L.stream_ptr())
    L.check(rc, "gemm_mxfp8")
    L.count_launches()
    return out


def usable(K: int, N: int) -> bool:
    """Both the forward (reduction over ``K``) and the input gradient (reduction over ``N``) need multiples of 128."""
    return K % 128 == 0 and N % 128 == 0


# Quantised copies of the expert weights, kept from one microbatch to the next.  A training engine that owns the weights switches
# the cache on and calls ``weights_changed()`` after every update (its kernels write the weights without touching their version
# counters); without an engine saying so nothing is cached.
_WEIGHT_CACHE: dict = {}
_WEIGHT_EPOCH = [0]
_CACHE_ON = [False]


def cache_weights(on: bool = True) -> None:
    _CACHE_ON[0] = bool(on)
    _WEIGHT_CACHE.clear()


def weights_changed() -> None:
    """Every weight may have changed (an optimizer step, a restore): quantised copies made before now are stale."""
    _WEIGHT_EPOCH[0] += 1
    _WEIGHT_CACHE.clear()


def _quantized_weight(w: torch.Tensor, transposed: bool, ident: int = 0):
    G_, N, K = w.shape
    key = (ident or id(w), w.data_ptr(), tuple(w.shape), transposed)
    stamp = (_WEIGHT_EPOCH[0], w._version)
    if _CACHE_ON[0]:
        hit = _WEIGHT_CACHE.get(key)
        if hit is not None and hit[0] == stamp:
            return hit[1], hit[2]
    if transposed:
        q, sc = quantize_mx(w.transpose(1, 2).contiguous().reshape(G_ * K, N), sf_rows=_pad128(G_ * K + TILE_N))
    else:
        q, sc = quantize_mx(w.reshape(G_ * N, K), sf_rows=_pad128(G_ * N + TILE_N))
    if _CACHE_ON[0]:
        _WEIGHT_CACHE[key] = (stamp, q, sc)
    return q, sc


class _MxGroupedLinear(torch.autograd.Function):
    """Expert projection ``x [rows, K]`` (expert-sorted, 128-aligned groups) by ``w [G, N, K]`` in MXFP8."""

    @staticmethod
    def forward(ctx, x, w, layout, out_holder=None, lean=False):
        # `out_holder`: a one-element list around the destination tensor (kept out of autograd's sight: the destination is fresh
        # memory to write, not an input whose history matters)
        out = out_holder[0] if out_holder else None
        ctx.layout, ctx.lean = layout, lean
        ctx.save_for_backward(x, w)
        ctx.ident = id(w)                  # (the backward sees an unpacked copy of the tensor object: the cache key stays the parameter's)
        G_, N, K = w.shape
        xq, xs = quantize_mx(x)
        wq, ws = _quantized_weight(w, False, ctx.ident)
        return gemm_mx(xq, xs, wq, ws, layout.tile_group, G_, out=out, zero_skipped=not lean)

    @staticmethod
    def backward(ctx, dy):
        from . import grouped as G
        from .functional import grad_accumulates
        x, w = ctx.saved_tensors
        layout = ctx.layout
        dy = dy.contiguous()
        G_, N, K = w.shape
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dX = dY W reduces over the output features: dY is quantised along N and so are the weights (transposed copy)
            dq, ds = quantize_mx(dy)
            wq, ws = _quantized_weight(w, True, ctx.ident)
            dx = gemm_mx(dq, ds, wq, ws, layout.tile_group, G_, zero_skipped=not ctx.lean)
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            if main is not None and dy.is_cuda:
                G.tgmm(dy, x, layout, G_, out=main, accumulate=grad_accumulates(w))
            else:
                dw = G.tgmm(dy, x, layout, G_).to(w.dtype)
        return dx, dw, None, None, None


def mx_grouped_linear(x, w, layout, out: Optional[torch.Tensor] = None, lean: bool = False):
    """``lean``: row tiles that hold no expert's rows are left unwritten instead of zero-filled (forward and input gradient); only for
    pipelines whose consumers never read those tiles (the expert-parallel exchange).  ``out``: the product is written there."""
    return _MxGroupedLinear.apply(x, w, layout, [out] if out is not None else None, lean)
