"""Token draws on the GPU: greedy argmax and temperature / top-k / min-p / top-p sampling, one CTA per row of logits
(``csrc/kernels/sampling.cu``).  The filters are thresholds found by radix descent (no sort); the draw is the inverse CDF
in token order at ``u * Z`` with ``u`` supplied by the caller, so keyed host generators keep deciding the stream.

Capability: src/dew/sampling/text.py (``Sampling``) and the serving draws of src/dew/inference/serving.py.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import library as L


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"logits must be fp32 or bf16, got {t.dtype}")


def kernel_ok(logits: torch.Tensor) -> bool:
    return (logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
            and L.use_cuda(logits) and hasattr(L.load(), "dewb_sample_rows"))


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """``logits [R, V] -> [R]`` int64, the lowest index among equal maxima."""
    if not kernel_ok(logits):
        return logits.argmax(-1)
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int64, device=logits.device)
    L.check(L.load().dewb_argmax_rows(L.ptr(logits), ctypes.c_int(_dtype_code(logits)), ctypes.c_longlong(R),
                                      ctypes.c_longlong(logits.stride(0)), ctypes.c_int(V), L.ptr(out), L.stream_ptr()), "argmax_rows")
    L.count_launches()
    return out


def filtered_reference(logits: torch.Tensor, temperature: float, top_k: Optional[int], top_p: float, min_p: float) -> torch.Tensor:
    """The scaled logits with everything the filters drop set to ``-inf`` (thresholds as the kernel takes them: ties at a
    threshold are kept)."""
    x = logits.float() / temperature
    V = x.shape[-1]
    keep = torch.ones_like(x, dtype=torch.bool)
    if top_k is not None and 0 < top_k < V:
        keep &= x >= torch.topk(x, top_k, dim=-1).values[:, -1:]
    if min_p > 0:
        keep &= x >= x.max(-1, keepdim=True).values + torch.log(torch.tensor(min_p, device=x.device))
    if top_p < 1.0:
        e = torch.where(keep, torch.exp(x - x.max(-1, keepdim=True).values), torch.zeros_like(x))
        z = e.sum(-1, keepdim=True)
        se, order = torch.sort(e, descending=True, dim=-1)
        above = se.cumsum(-1) - se                               # mass of strictly earlier entries in sorted order
        xs = x.gather(-1, order)
        # mass of strictly greater logits: the first occurrence of each value in sorted order carries it
        first = torch.ones_like(xs, dtype=torch.bool)
        first[:, 1:] = xs[:, 1:] != xs[:, :-1]
        above_val = torch.where(first, above, torch.zeros_like(above)).cummax(-1).values
        keep_sorted = above_val < top_p * z
        keep &= torch.zeros_like(keep).scatter(-1, order, keep_sorted)
    return x.masked_fill(~keep, float("-inf"))


def sample_rows(logits: torch.Tensor, uniform: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None, top_p: float = 1.0,
                min_p: float = 0.0, return_kept: bool = False):
    """One token per row of ``logits [R, V]`` from ``softmax(filter(logits / temperature))``; ``uniform [R]`` in ``[0, 1)``."""
    R, V = logits.shape
    if not kernel_ok(logits):
        x = filtered_reference(logits, temperature, top_k, top_p, min_p)
        e = torch.exp(x - x.max(-1, keepdim=True).values)
        cdf = e.cumsum(-1)
        tok = torch.searchsorted(cdf, (uniform.to(cdf) * cdf[:, -1]).unsqueeze(-1), right=True).squeeze(-1).clamp_max(V - 1)
        return (tok, torch.isfinite(x).sum(-1).int()) if return_kept else tok
    out = torch.empty(R, dtype=torch.int64, device=logits.device)
    kept = torch.empty(R, dtype=torch.int32, device=logits.device) if return_kept else None
    u = uniform.to(device=logits.device, dtype=torch.float32).contiguous()
    L.check(L.load().dewb_sample_rows(L.ptr(logits), ctypes.c_int(_dtype_code(logits)), ctypes.c_longlong(R),
                                      ctypes.c_longlong(logits.stride(0)), ctypes.c_int(V), L.ptr(u), ctypes.c_float(temperature),
                                      ctypes.c_int(int(top_k) if top_k else 0), ctypes.c_float(top_p), ctypes.c_float(min_p),
                                      L.ptr(out), L.ptr(kept), L.stream_ptr()), "sample_rows")
    L.count_launches()
    return (out, kept) if return_kept else out
