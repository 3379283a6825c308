"""Attention dispatch on the GPU: the sm_100a flash kernels or the library arm (cuDNN / flash SDPA via torch).

The selector records, per call, which kernel ran and why the other refused (``explain``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import library as L
from .selection import Kernel, Requirement, op

_ATTN = op("attention")


def _flash_available() -> bool:
    try:
        return hasattr(L.load(), "dewb_flash_fwd")
    except Exception:
        return False


def _bwd_available() -> bool:
    from .flash import bwd_available
    return bwd_available()


_ATTN.kernels = [
    Kernel("sm100_flash", [
        Requirement("built", lambda c: _flash_available(), "flash kernels are not in this build of libdewb.so"),
        Requirement("dtype", lambda c: c["dtype"] == torch.bfloat16, "bf16 only"),
        Requirement("head_dim", lambda c: c["D"] in (64, 128), "head_dim must be 64 or 128"),
        Requirement("variants", lambda c: not c["segments"] or (c["S"] == c["T"] and c["S"] % 4 == 0),
                    "packed segments need S == T and rows of ids on 16-byte boundaries"),
        Requirement("seq", lambda c: c["S"] == c["T"] and c["S"] % 128 == 0, "needs S == T and S a multiple of 128"),
        Requirement("gqa", lambda c: c["Hq"] % c["Hkv"] == 0, "query heads must be a multiple of kv heads"),
        Requirement("backward", lambda c: not c["grad"] or _bwd_available(), "the backward kernels are not in this build"),
        Requirement("layout", lambda c: c["unit_d"], "head_dim must have unit stride"),
    ], receipt="tcgen05 flash forward/backward, csrc/kernels/flash_sm100.cu"),
    Kernel("sdpa", [], receipt="library arm: torch scaled_dot_product_attention (cuDNN / flash)"),
]


def _sdpa(q, k, v, causal, scale, window, softcap, sinks, segment_ids):
    if window is not None or softcap or sinks is not None or segment_ids is not None:
        from .functional import attention_reference
        if q.is_cuda and q.shape[1] >= 2048:
            import warnings
            warnings.warn("attention with a window / soft-cap / sinks / packed segments that the sm_100a kernel refused runs "
                          f"the O(S^2)-memory PyTorch path on the GPU (S = {q.shape[1]})", stacklevel=3)
        return attention_reference(q, k, v, causal, scale, window, softcap, sinks, segment_ids)
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    o = F.scaled_dot_product_attention(qh, kh, vh, is_causal=causal and q.shape[1] > 1, scale=scale,
                                       enable_gqa=q.shape[2] != k.shape[2])
    return o.transpose(1, 2)


def flash_attention(q, k, v, causal=True, scale=None, window=None, softcap=0.0, sinks=None, segment_ids=None,
                    kernel: Optional[str] = None):
    B, S, Hq, D = q.shape
    case = dict(dtype=q.dtype, D=D, S=S, T=k.shape[1], Hq=Hq, Hkv=k.shape[2], sinks=sinks is not None,
                softcap=bool(softcap), window=window, segments=segment_ids is not None, causal=causal,
                grad=torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad),
                unit_d=q.stride(3) == 1 and k.stride(3) == 1 and v.stride(3) == 1)
    which = _ATTN.select(case, forced=kernel)
    if which == "sm100_flash":
        from .flash import flash_sm100
        return flash_sm100(q, k, v, causal, scale if scale is not None else 1.0 / math.sqrt(D), window=window,
                           softcap=softcap, sinks=sinks, segment_ids=segment_ids)
    return _sdpa(q, k, v, causal, scale, window, softcap, sinks, segment_ids)


def packed_attention(qkv, cos, sin, positions, Hq: int, Hkv: int, causal: bool = True, scale: Optional[float] = None):
    """RoPE + attention over a packed projection ``[B, S, Hq + 2 Hkv, D]`` when the sm_100a flash kernels take the case
    (one fused autograd node, no slice copies); returns None when they do not, and the caller takes the general path."""
    B, S, H, D = qkv.shape
    if not (L.use_cuda(qkv) and qkv.is_contiguous()):
        return None
    case = dict(dtype=qkv.dtype, D=D, S=S, T=S, Hq=Hq, Hkv=Hkv, sinks=False, softcap=False, window=None, segments=False,
                causal=causal, grad=torch.is_grad_enabled() and qkv.requires_grad, unit_d=True)
    if _ATTN.select(case) != "sm100_flash":
        return None
    from .flash import packed_rope_flash
    return packed_rope_flash(qkv, cos, sin, positions, Hq, Hkv, causal, scale if scale is not None else 1.0 / math.sqrt(D))
