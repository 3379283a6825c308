"""Mamba-2 SSD on the sm_100a scan kernel (``csrc/kernels/ssd_sm100.cu``): state dimension 128, head dimension 64, heads
taken in pairs of one B / C group.

Forward: the per-head decayed score blocks ``P_h = (C B^T) o e^{g_i - g_j}`` and the running log decay ``g`` are prepared as
batched products, then ONE sequential kernel per (batch, head pair) walks the chunks with the state in registers / a bf16
operand tile (see the kernel's header).  Backward: the loop-free chunked form in PyTorch (``ops.scan.ssd_chunked``) is
re-evaluated under autograd.  Reference: src/dew/nn/kernels/mamba_ssd.py (ChunkCumsum, BmmChunk, ChunkState, StatePassing,
ChunkScan), src/dew/nn/mixers/mamba2.py:101 ``chunk_ssd``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import library as L

CHUNK = 64


def kernel_available(x: torch.Tensor, Bm: torch.Tensor) -> bool:
    H, P = x.shape[2], x.shape[3]
    G, N = Bm.shape[2], Bm.shape[3]
    return (x.is_cuda and P == 64 and N == 128 and H % 2 == 0 and H % G == 0 and (H // G) % 2 == 0 and L.exists()
            and hasattr(L.load(), "dewb_ssd_scan_fwd"))


def prepare(x, dt, A, Bm, Cm):
    """-> xdt bf16 ``[B,T,H,P]``, Bm / Cm bf16, P bf16 ``[B*H, Tp, 64]``, gc fp32 ``[B*H, Tp]``."""
    B, T, H, P = x.shape
    G = Bm.shape[2]
    Tp = (T + CHUNK - 1) // CHUNK * CHUNK
    Nc = Tp // CHUNK
    pad = Tp - T
    dtf = dt.float()
    a = torch.nn.functional.pad(dtf * A.float(), (0, 0, 0, pad))                            # [B,Tp,H]
    gc = a.reshape(B, Nc, CHUNK, H).cumsum(2)                                               # [B,Nc,C,H]
    xdt = (x.float() * dtf[..., None]).to(torch.bfloat16).contiguous()
    b16, c16 = Bm.to(torch.bfloat16).contiguous(), Cm.to(torch.bfloat16).contiguous()
    bc = torch.nn.functional.pad(b16, (0, 0, 0, 0, 0, pad)).reshape(B, Nc, CHUNK, G, -1)
    cc = torch.nn.functional.pad(c16, (0, 0, 0, 0, 0, pad)).reshape(B, Nc, CHUNK, G, -1)
    cb = torch.einsum("bcign,bcjgn->bcgij", cc, bc).float()                                 # [B,Nc,G,C,C]
    g_h = gc.permute(0, 1, 3, 2)                                                            # [B,Nc,H,C]
    diff = g_h[..., :, None] - g_h[..., None, :]
    tril = torch.tril(torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=x.device))
    decay = torch.where(tril, torch.exp(torch.where(tril, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    Pm = (cb.repeat_interleave(H // G, 2) * decay).to(torch.bfloat16)                       # [B,Nc,H,C,C]
    Pm = Pm.permute(0, 2, 1, 3, 4).reshape(B * H, Tp, CHUNK).contiguous()
    gcf = g_h.permute(0, 2, 1, 3).reshape(B * H, Tp).contiguous()
    return xdt, b16, c16, Pm, gcf, Tp


def scan_cuda(xdt, b16, c16, Pm, gc, Tp: int, initial_state: Optional[torch.Tensor]):
    B, T, H, P = xdt.shape
    G = b16.shape[2]
    dev = xdt.device
    out = torch.empty(B, T, H, P, dtype=torch.bfloat16, device=dev)
    final = torch.empty(B, H, P, b16.shape[3], dtype=torch.float32, device=dev)
    init = None if initial_state is None else initial_state.float().contiguous()
    L.ensure_device(xdt)
    rc = L.load().dewb_ssd_scan_fwd(L.ptr(xdt), L.ptr(b16), L.ptr(c16), L.ptr(Pm), L.ptr(gc), L.ptr(init), L.ptr(out), L.ptr(final),
                                    ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(G), ctypes.c_int(Tp),
                                    L.ptr(L.status(dev)), L.stream_ptr())
    L.check(rc, "ssd_scan_fwd")
    L.count_launches()
    return out, final


class _SSD(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A, Bm, Cm, D, initial_state):
        ctx.save_for_backward(x, dt, A, Bm, Cm, D, initial_state)
        xdt, b16, c16, Pm, gc, Tp = prepare(x, dt, A, Bm, Cm)
        y, S = scan_cuda(xdt, b16, c16, Pm, gc, Tp, initial_state)
        if D is not None:
            y = (y.float() + x.float() * D.float()[None, None, :, None]).to(y.dtype)
        return y.to(x.dtype), S

    @staticmethod
    def backward(ctx, dy, dS):
        from .scan import ssd_chunked
        saved = ctx.saved_tensors
        with torch.enable_grad():
            leaves = [None if t is None else t.detach().requires_grad_(t.is_floating_point()) for t in saved]
            y, S = ssd_chunked(*leaves)
            need = [(t, i) for i, t in enumerate(leaves) if t is not None and ctx.needs_input_grad[i]]
            grads = torch.autograd.grad((y, S), [t for t, _ in need], (dy.to(y.dtype), dS.to(S.dtype)), allow_unused=True)
        out = [None] * 7
        for (t, i), g in zip(need, grads):
            out[i] = g
        return tuple(out)


def ssd(x, dt, A, Bm, Cm, D=None, initial_state=None):
    """x ``[B,T,H,64]``, dt ``[B,T,H]`` (after softplus), A ``[H]``, B / C ``[B,T,G,128]`` -> (y ``[B,T,H,64]``, state
    ``[B,H,64,128]`` fp32)."""
    return _SSD.apply(x, dt, A, Bm, Cm, D, initial_state)
