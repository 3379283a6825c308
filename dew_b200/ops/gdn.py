"""Gated delta rule on the sm_100a kernels (``csrc/kernels/gdn_sm100.cu``): three launches per forward or backward.

``prepare``   chunk-parallel, one CTA per 128 tokens of one (batch, head): within-chunk cumulative log decay, ``K K^T`` and
              ``Q K^T`` on the tensor cores, the strictly lower system ``(I + A) [W | U] = [beta e^g K | beta V]`` solved by
              forward substitution in fp32, the masked decayed scores ``P`` and (for the backward) ``e^g Q``.
``scan_fwd``  sequential over chunks, one CTA per (batch, head), the ``[Dk, Dv]`` state in fp32 registers and as a bf16
              operand tile in shared memory: ``Vn = U - W S``; ``O = e^g Q S + P Vn``; ``S <- e^{g_L} S + (e^{g_L - g} K)^T Vn``.
``scan_bwd``  the same walk in reverse for the state gradient: ``dVn = P^T dO + e^{g_L - g} K dS``;
              ``dS <- e^{g_L} dS + (e^g Q)^T dO - W^T dVn``; it leaves every chunk's exit-state gradient in memory.

The remaining gradients are local to a chunk once its entry state and exit-state gradient are known; they are taken by
differentiating the chunk-local formula, batched over all chunks (``_chunk_local``).  Every stage has a PyTorch
restatement here (``*_reference``) that serves as the oracle for the kernels and as the CPU path.

Replaces src/dew/nn/kernels/fla_gdn.py (``KktSolve``, ``RecomputeWU``, ``ChunkFwdH``, ``ChunkFwdO``, ``ChunkBwdDhu``) and the
recurrence template's chunked forward (src/dew/nn/kernels/templates/recurrence/chunk_forward.py).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import library as L

CHUNK = 64
PAIR = 128          # tokens per prepare CTA
HEAD_DIM = 128      # the kernels are built for 128-wide keys and values


def padded_len(T: int) -> int:
    return (T + PAIR - 1) // PAIR * PAIR


def kernel_available(q: torch.Tensor, v: torch.Tensor) -> bool:
    return (q.is_cuda and q.shape[-1] == HEAD_DIM and v.shape[-1] == HEAD_DIM and L.exists()
            and hasattr(L.load(), "dewb_gdn_scan_fwd"))


# ---------------------------------------------------------------------------------------------------------------
# PyTorch restatements of the three stages (oracle and CPU path).  Layouts match the kernels'.


def prepare_reference(q, k, v, g, beta, scale: float, round_bf16: bool = False):
    """q, k, v ``[B,T,H,D]``; g, beta ``[B,T,H]`` -> gc ``[X,Tp]``, W ``[X,Tp,Dk]``, U ``[X,Tp,Dv]``, P ``[X,Tp,64]``,
    Qg ``[X,Tp,Dk]`` with ``X = B*H`` and ``Tp`` the length padded to 128."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    Tp = padded_len(T)
    f = torch.float64 if q.dtype == torch.float64 else torch.float32
    pad = Tp - T
    tr = lambda x: torch.nn.functional.pad(x.to(f).permute(0, 2, 1, 3).reshape(B * H, T, -1), (0, 0, 0, pad))
    qf, kf, vf = tr(q), tr(k), tr(v)
    tr1 = lambda x: torch.nn.functional.pad(x.to(f).permute(0, 2, 1).reshape(B * H, T), (0, pad))
    gf, bf = tr1(g), tr1(beta)
    X, N = B * H, Tp // CHUNK
    c = lambda x: x.reshape(X, N, CHUNK, *x.shape[2:])
    qc, kc, vc, gc, bc = c(qf), c(kf), c(vf), c(gf).cumsum(-1), c(bf)
    diff = gc[..., :, None] - gc[..., None, :]
    incl = torch.tril(torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=q.device))
    strict = torch.tril(torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=q.device), -1)
    decay = torch.exp(torch.where(incl, diff, torch.zeros_like(diff)))
    A = torch.where(strict, bc[..., None] * (kc @ kc.transpose(-1, -2)) * decay, torch.zeros_like(decay))
    eye = torch.eye(CHUNK, dtype=f, device=q.device)
    rhs = torch.cat([kc * (bc * gc.exp())[..., None], vc * bc[..., None]], -1)
    sol = torch.linalg.solve_triangular(eye + A, rhs, upper=False)
    W, U = sol[..., :Dk], sol[..., Dk:]
    P = torch.where(incl, scale * (qc @ kc.transpose(-1, -2)) * decay, torch.zeros_like(decay))
    Qg = qc * (scale * gc.exp())[..., None]
    flat = lambda x: x.reshape(X, Tp, *x.shape[3:])
    outs = [flat(gc), flat(W), flat(U), flat(P), flat(Qg)]
    if round_bf16:
        outs = [outs[0]] + [o.to(torch.bfloat16).to(f) for o in outs[1:]]
    return tuple(outs)


def scan_fwd_reference(q, k, gc, W, U, P, scale: float, initial_state=None, save_states: bool = False):
    """-> o ``[B,T,H,Dv]``, final state ``[X,Dk,Dv]``, chunk-entry states ``[X,N,Dk,Dv]`` (or None)."""
    B, T, H, Dk = q.shape
    X, Tp, Dv = U.shape
    N = (T + CHUNK - 1) // CHUNK
    f = W.dtype
    pad = Tp - T
    tr = lambda x: torch.nn.functional.pad(x.to(f).permute(0, 2, 1, 3).reshape(X, T, -1), (0, 0, 0, pad))
    qf, kf = tr(q), tr(k)
    S = torch.zeros(X, Dk, Dv, dtype=f, device=q.device) if initial_state is None else initial_state.reshape(X, Dk, Dv).to(f).clone()
    outs, states = [], []
    for n in range(N):
        sl = slice(n * CHUNK, (n + 1) * CHUNK)
        gi = gc[:, sl]
        gl = gi[:, -1]
        if save_states:
            states.append(S.clone())
        Vn = U[:, sl] - W[:, sl] @ S
        o = (scale * gi.exp())[..., None] * (qf[:, sl] @ S) + P[:, sl] @ Vn
        outs.append(o)
        S = S * gl.exp()[:, None, None] + (kf[:, sl] * (gl[:, None] - gi).exp()[..., None]).transpose(-1, -2) @ Vn
    o = torch.cat(outs, 1)[:, :T].reshape(B, H, T, Dv).permute(0, 2, 1, 3)
    return o, S, (torch.stack(states, 1) if save_states else None)


def scan_bwd_reference(do, k, gc, W, P, Qg, d_final=None):
    """-> exit-state gradients per chunk ``[X,N,Dk,Dv]`` and the gradient of the initial state ``[X,Dk,Dv]``."""
    B, T, H, Dv = do.shape
    X, Tp, Dk = W.shape
    N = (T + CHUNK - 1) // CHUNK
    f = W.dtype
    pad = Tp - T
    tr = lambda x: torch.nn.functional.pad(x.to(f).permute(0, 2, 1, 3).reshape(X, T, -1), (0, 0, 0, pad))
    dof, kf = tr(do), tr(k)
    dS = torch.zeros(X, Dk, Dv, dtype=f, device=do.device) if d_final is None else d_final.reshape(X, Dk, Dv).to(f).clone()
    out = [None] * N
    for n in range(N - 1, -1, -1):
        sl = slice(n * CHUNK, (n + 1) * CHUNK)
        gi = gc[:, sl]
        gl = gi[:, -1]
        out[n] = dS.clone()
        dVn = P[:, sl].transpose(-1, -2) @ dof[:, sl] + (gl[:, None] - gi).exp()[..., None] * (kf[:, sl] @ dS)
        dS = dS * gl.exp()[:, None, None] + Qg[:, sl].transpose(-1, -2) @ dof[:, sl] - W[:, sl].transpose(-1, -2) @ dVn
    return torch.stack(out, 1), dS


def _chunk_local(qc, kc, vc, gr, bc, S0, scale: float):
    """One chunk's outputs as a differentiable function of its own inputs and its entry state, batched over chunks:
    qc, kc ``[Y,64,Dk]``, vc ``[Y,64,Dv]``, gr (raw log decay), bc ``[Y,64]``, S0 ``[Y,Dk,Dv]`` -> (O ``[Y,64,Dv]``, S1)."""
    gc = gr.cumsum(-1)
    diff = gc[..., :, None] - gc[..., None, :]
    incl = torch.tril(torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=qc.device))
    strict = torch.tril(torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=qc.device), -1)
    decay = torch.exp(torch.where(incl, diff, torch.zeros_like(diff)))
    kk = kc @ kc.transpose(-1, -2)
    A = torch.where(strict, bc[..., None] * kk * decay, torch.zeros_like(decay))
    eye = torch.eye(CHUNK, dtype=qc.dtype, device=qc.device)
    rhs = torch.cat([kc * (bc * gc.exp())[..., None], vc * bc[..., None]], -1)
    sol = torch.linalg.solve_triangular(eye + A, rhs, upper=False)
    Dk = qc.shape[-1]
    W, U = sol[..., :Dk], sol[..., Dk:]
    Vn = U - W @ S0
    P = torch.where(incl, scale * (qc @ kc.transpose(-1, -2)) * decay, torch.zeros_like(decay))
    O = (scale * gc.exp())[..., None] * (qc @ S0) + P @ Vn
    gl = gc[..., -1]
    S1 = S0 * gl.exp()[:, None, None] + (kc * (gl[:, None] - gc).exp()[..., None]).transpose(-1, -2) @ Vn
    return O, S1


def chunk_local_grads(q, k, v, g, beta, states, dstates, do, scale: float, slab_chunks: int = 4096, analytic: bool = True):
    """Gradients of q, k, v, g, beta given every chunk's entry state and exit-state gradient; fp32, batched in slabs of
    chunks so the temporaries stay bounded."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    N = (T + CHUNK - 1) // CHUNK
    Tc = N * CHUNK
    pad = Tc - T
    f = torch.float64 if q.dtype == torch.float64 else torch.float32
    X = B * H
    tr = lambda x: torch.nn.functional.pad(x.to(f).permute(0, 2, 1, 3).reshape(X, T, -1), (0, 0, 0, pad)).reshape(X * N, CHUNK, -1)
    tr1 = lambda x: torch.nn.functional.pad(x.to(f).permute(0, 2, 1).reshape(X, T), (0, pad)).reshape(X * N, CHUNK)
    qc, kc, vc, doc = tr(q), tr(k), tr(v), tr(do)
    gr, bc = tr1(g), tr1(beta)
    S0 = states.reshape(X * N, Dk, Dv)
    dS1 = dstates.reshape(X * N, Dk, Dv)
    grads = [torch.empty_like(t) for t in (qc, kc, vc, gr, bc)]
    Y = X * N
    for a in range(0, Y, slab_chunks):
        sl = slice(a, min(Y, a + slab_chunks))
        if analytic:
            res = _chunk_local_analytic(qc[sl], kc[sl], vc[sl], gr[sl], bc[sl], S0[sl].to(f), doc[sl], dS1[sl].to(f), scale)
        else:
            ins = [t[sl].detach().requires_grad_(True) for t in (qc, kc, vc, gr, bc)]
            with torch.enable_grad():
                O, S1 = _chunk_local(*ins, S0[sl].to(f), scale)
                res = torch.autograd.grad((O, S1), ins, (doc[sl], dS1[sl].to(f)))
        for dst, r in zip(grads, res):
            dst[sl] = r
    back = lambda x, D: x.reshape(X, Tc, D)[:, :T].reshape(B, H, T, D).permute(0, 2, 1, 3)
    back1 = lambda x: x.reshape(X, Tc)[:, :T].reshape(B, H, T).permute(0, 2, 1)
    return back(grads[0], Dk), back(grads[1], Dk), back(grads[2], Dv), back1(grads[3]), back1(grads[4])


def _chunk_local_analytic(qc, kc, vc, gr, bc, S0, dO, dS1, scale: float):
    """Closed-form gradients of one chunk (batched over chunks), the same quantities ``torch.autograd`` gives for
    ``_chunk_local``.  With ``M = I + A``, ``T = M^-1``, ``W = T (beta e^g K)``, ``U = T (beta V)``:

        dVn = P^T dO + Kd dS1                      dW = -dVn S0^T,  dU = dVn
        dQ  = scale e^g (dO S0^T) + (dP o D) K     dP = tril(dO Vn^T) (scale folded into ``Gt = scale dP o D``)
        dKt = T^T dW, dVt = T^T dU                 dA = -strict(dKt W^T + dVt U^T)
        dK  = Gt^T Q + e^{g_L - g} (Vn dS1^T) + beta e^g dKt + Bt K + Bt^T K      with Bt = dA o (beta_i D_ij)
        dV  = beta dVt
    and the decay / write-strength gradients collect the row sums of the same products."""
    gc = gr.cumsum(-1)
    eg = gc.exp()
    gl = gc[..., -1:]
    diff = gc[..., :, None] - gc[..., None, :]
    incl = torch.tril(torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=qc.device))
    strict = torch.tril(torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=qc.device), -1)
    zero = torch.zeros_like(diff)
    D = torch.where(incl, torch.exp(torch.where(incl, diff, zero)), zero)
    kk = kc @ kc.transpose(-1, -2)
    kkD = torch.where(strict, kk * D, zero)
    A = bc[..., None] * kkD
    eye = torch.eye(CHUNK, dtype=qc.dtype, device=qc.device)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
    Kt = kc * (bc * eg)[..., None]
    W, U = Tm @ Kt, Tm @ (vc * bc[..., None])
    Vn = U - W @ S0
    qk = qc @ kc.transpose(-1, -2)
    P = scale * qk * D
    tail = (gl - gc).exp()                                    # e^{g_L - g}
    Kd = kc * tail[..., None]
    dVn = P.transpose(-1, -2) @ dO + Kd @ dS1
    S0t = S0.transpose(-1, -2)
    dQ1 = (scale * eg)[..., None] * (dO @ S0t)
    Gt = scale * torch.where(incl, dO @ Vn.transpose(-1, -2), zero) * D
    dQ = dQ1 + Gt @ kc
    dKd = Vn @ dS1.transpose(-1, -2)
    dW = -(dVn @ S0t)
    Tt = Tm.transpose(-1, -2)
    dKt, dVt = Tt @ dW, Tt @ dVn
    dA = -torch.where(strict, dKt @ W.transpose(-1, -2) + dVt @ U.transpose(-1, -2), zero)
    Bt = dA * bc[..., None] * D
    dK = Gt.transpose(-1, -2) @ qc + tail[..., None] * dKd + (bc * eg)[..., None] * dKt + Bt @ kc + Bt.transpose(-1, -2) @ kc
    dV = bc[..., None] * dVt
    dbeta = (dVt * vc).sum(-1) + eg * (dKt * kc).sum(-1) + (dA * kkD).sum(-1)
    E = dA * A
    GP = Gt * qk                                              # dP o P
    kdk = (dKd * Kd).sum(-1)
    dgc = (dQ1 * qc).sum(-1) + GP.sum(-1) - GP.sum(-2) - kdk + (dKt * Kt).sum(-1) + E.sum(-1) - E.sum(-2)
    dgl = kdk.sum(-1) + gl[..., 0].exp() * (dS1 * S0).sum((-1, -2))
    dgc = torch.cat([dgc[..., :-1], (dgc[..., -1] + dgl)[..., None]], -1)
    dg = dgc.flip(-1).cumsum(-1).flip(-1)
    return dQ, dK, dV, dg, dbeta


# ---------------------------------------------------------------------------------------------------------------
# kernel launchers


def _strides3(t):
    assert t.stride(-1) == 1
    return [ctypes.c_longlong(t.stride(0)), ctypes.c_longlong(t.stride(1)), ctypes.c_longlong(t.stride(2))]


def prepare_cuda(q, k, v, g, beta, scale: float, want_qg: bool):
    """q, k may carry fewer heads than v (``rep = Hv / Hk`` consecutive value heads share a key head)."""
    B, T, H, _ = v.shape
    rep = H // q.shape[2]
    X, Tp = B * H, padded_len(T)
    dev = q.device
    gc = torch.empty(X, Tp, dtype=torch.float32, device=dev)
    W = torch.empty(X, Tp, HEAD_DIM, dtype=torch.bfloat16, device=dev)
    U = torch.empty_like(W)
    P = torch.empty(X, Tp, CHUNK, dtype=torch.bfloat16, device=dev)
    Qg = torch.empty_like(W) if want_qg else None
    lib = L.load()
    L.ensure_device(q)
    rc = lib.dewb_gdn_prepare(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta), L.ptr(gc), L.ptr(W), L.ptr(U), L.ptr(P),
                              L.ptr(Qg), ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(rep), *_strides3(q), *_strides3(k),
                              *_strides3(v), ctypes.c_float(scale), L.ptr(L.status(dev)), L.stream_ptr())
    L.check(rc, "gdn_prepare")
    L.count_launches()
    return gc, W, U, P, Qg


def scan_fwd_cuda(q, k, gc, W, U, P, scale: float, initial_state, save_states: bool, save_vn: bool = False):
    B, T = q.shape[:2]
    X, Tp = W.shape[0], gc.shape[1]
    H = X // B
    rep = H // q.shape[2]
    N = (T + CHUNK - 1) // CHUNK
    dev = q.device
    o = torch.empty(B, T, H, HEAD_DIM, dtype=torch.bfloat16, device=dev)
    final = torch.empty(X, HEAD_DIM, HEAD_DIM, dtype=torch.float32, device=dev)
    states = torch.empty(X, N, HEAD_DIM, HEAD_DIM, dtype=torch.bfloat16, device=dev) if save_states else None
    vn = None
    if save_vn:
        vn = torch.empty(X, Tp, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        vn[:, N * CHUNK:].zero_()                      # the chunk the padding to 128 adds is never visited
    init = None if initial_state is None else initial_state.reshape(X, HEAD_DIM, HEAD_DIM).float().contiguous()
    lib = L.load()
    L.ensure_device(q)
    rc = lib.dewb_gdn_scan_fwd(L.ptr(q), L.ptr(k), L.ptr(gc), L.ptr(W), L.ptr(U), L.ptr(P), L.ptr(init), L.ptr(o), L.ptr(final),
                               L.ptr(states), L.ptr(vn), ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(rep), ctypes.c_int(Tp),
                               *_strides3(q), *_strides3(k), ctypes.c_float(scale), L.ptr(L.status(dev)), L.stream_ptr())
    L.check(rc, "gdn_scan_fwd")
    L.count_launches()
    # the kernel stores each chunk-entry state transposed ([Dv, Dk], the operand tile it keeps in shared memory)
    if save_vn:
        return o, final, states, vn                     # raw layouts, as the backward kernels read them
    return o, final, (states.transpose(-1, -2) if save_states else None)


def scan_bwd_cuda(do, k, gc, W, P, Qg, d_final, for_kernels: bool = False):
    B, T, H, _ = do.shape
    X, Tp = B * H, gc.shape[1]
    rep = H // k.shape[2]
    N = (T + CHUNK - 1) // CHUNK
    dev = do.device
    dstates = None if for_kernels else torch.empty(X, N, HEAD_DIM, HEAD_DIM, dtype=torch.float32, device=dev)
    dstates16 = dvn = None
    if for_kernels:
        dstates16 = torch.empty(X, N, HEAD_DIM, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        dvn = torch.empty(X, Tp, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        dvn[:, N * CHUNK:].zero_()
    d_init = torch.empty(X, HEAD_DIM, HEAD_DIM, dtype=torch.float32, device=dev)
    dfin = None if d_final is None else d_final.reshape(X, HEAD_DIM, HEAD_DIM).float().contiguous()
    lib = L.load()
    L.ensure_device(do)
    rc = lib.dewb_gdn_scan_bwd(L.ptr(do), L.ptr(k), L.ptr(gc), L.ptr(W), L.ptr(P), L.ptr(Qg), L.ptr(dfin), L.ptr(dstates),
                               L.ptr(dstates16), L.ptr(dvn), L.ptr(d_init), ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(rep),
                               ctypes.c_int(Tp),
                               *_strides3(do), *_strides3(k), L.ptr(L.status(dev)), L.stream_ptr())
    L.check(rc, "gdn_scan_bwd")
    L.count_launches()
    if for_kernels:
        return dstates16, dvn, d_init
    return dstates, d_init


def local_bwd_cuda(q, k, v, do, gc, beta, W, U, P, vn, dvn, states_raw, dstates16, scale: float):
    """The chunk-local gradients on the two backward kernels (``csrc/kernels/gdn_bwd_sm100.cu``): dq, dk, dv (bf16) and
    dg, dbeta (fp32), from the intermediates the prepare kernel and the two scans leave in memory."""
    B, T, H, _ = v.shape
    rep = H // q.shape[2]
    X, Tp = B * H, gc.shape[1]
    N = (T + CHUNK - 1) // CHUNK
    dev = q.device
    bf = dict(dtype=torch.bfloat16, device=dev)
    dKt, dVt = torch.empty(X, Tp, HEAD_DIM, **bf), torch.empty(X, Tp, HEAD_DIM, **bf)
    if N * CHUNK < Tp:
        dKt[:, N * CHUNK:].zero_()
        dVt[:, N * CHUNK:].zero_()
    dq_part = torch.empty(B, T, H, HEAD_DIM, dtype=torch.float32, device=dev)
    dk_part = torch.empty_like(dq_part)
    gpart = torch.empty(X, Tp, dtype=torch.float32, device=dev)
    bpart = torch.empty_like(gpart)
    dq, dk, dv = (torch.empty(B, T, H, HEAD_DIM, **bf) for _ in range(3))
    dg = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    dbeta = torch.empty_like(dg)
    L.ensure_device(q)
    rc = L.load().dewb_gdn_bwd_local(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(do), L.ptr(vn), L.ptr(dvn), L.ptr(W), L.ptr(U), L.ptr(P),
                                     L.ptr(gc), L.ptr(beta), L.ptr(states_raw), L.ptr(dstates16), L.ptr(dKt), L.ptr(dVt),
                                     L.ptr(dq_part), L.ptr(dk_part), L.ptr(gpart), L.ptr(bpart), L.ptr(dq), L.ptr(dk), L.ptr(dv),
                                     L.ptr(dg), L.ptr(dbeta), ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(rep), ctypes.c_int(Tp),
                                     ctypes.c_float(scale), L.ptr(L.status(dev)), L.stream_ptr())
    L.check(rc, "gdn_bwd_local")
    L.count_launches(2)
    if rep > 1:                      # the kernels return dq, dk per value head: sum each group of `rep`
        Hk = H // rep
        dq = dq.view(B, T, Hk, rep, HEAD_DIM).float().sum(3).to(torch.bfloat16)
        dk = dk.view(B, T, Hk, rep, HEAD_DIM).float().sum(3).to(torch.bfloat16)
    return dq, dk, dv, dg, dbeta


def local_kernels_available() -> bool:
    import os
    return hasattr(L.load(), "dewb_gdn_bwd_local") and os.environ.get("DEWB_GDN_LOCAL", "kernel") != "torch"


# ---------------------------------------------------------------------------------------------------------------
# autograd node


def _stages(q):
    if q.is_cuda and not L.use_cuda(q):
        raise L.LibraryMissing("gated delta rule: CUDA tensors need the kernel library")
    return q.is_cuda


class _GatedDeltaRule(torch.autograd.Function):
    """Forward: prepare + forward scan.  Backward: prepare and forward scan again (keeping the chunk-entry states this
    time - nothing but the inputs is saved between the passes), reverse scan, chunk-local gradients."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, initial_state, scale):
        ctx.scale = scale
        ctx.has_initial = initial_state is not None
        ctx.save_for_backward(q, k, v, g, beta, initial_state)
        B, T, H, Dk = v.shape[0], v.shape[1], v.shape[2], q.shape[3]
        if not q.is_cuda and q.shape[2] != H:
            raise ValueError("shared key heads are a kernel-path feature: repeat q and k over the value heads on the CPU path")
        if _stages(q):
            gc, W, U, P, _ = prepare_cuda(q, k, v, g, beta, scale, False)
            o, final, _ = scan_fwd_cuda(q, k, gc, W, U, P, scale, initial_state, False)
        else:
            gc, W, U, P, _ = prepare_reference(q, k, v, g, beta, scale)
            o, final, _ = scan_fwd_reference(q, k, gc, W, U, P, scale, initial_state, False)
            o = o.to(v.dtype)
        return o, final.reshape(B, H, Dk, v.shape[-1])

    @staticmethod
    def backward(ctx, do, dfinal):
        q, k, v, g, beta, initial_state = ctx.saved_tensors
        scale = ctx.scale
        B, T, H, Dk = v.shape[0], v.shape[1], v.shape[2], q.shape[3]
        Dv = v.shape[-1]
        if _stages(q) and local_kernels_available():
            do = do.contiguous().to(torch.bfloat16)
            gc, W, U, P, Qg = prepare_cuda(q, k, v, g, beta, scale, True)
            _, _, states_raw, vn = scan_fwd_cuda(q, k, gc, W, U, P, scale, initial_state, True, save_vn=True)
            dstates16, dvn, d_init = scan_bwd_cuda(do, k, gc, W, P, Qg, dfinal, for_kernels=True)
            dq, dk, dv, dg, dbeta = local_bwd_cuda(q, k, v, do, gc, beta, W, U, P, vn, dvn, states_raw, dstates16, scale)
            d_init = d_init.reshape(B, H, Dk, Dv).to(initial_state.dtype) if ctx.has_initial else None
            return dq, dk, dv, dg.to(g.dtype), dbeta.to(beta.dtype), d_init, None
        rep = H // q.shape[2]
        q_in, k_in = q, k
        if rep > 1:                  # the PyTorch chunk-local path works per value head
            q, k = q.repeat_interleave(rep, 2), k.repeat_interleave(rep, 2)
        if _stages(q):
            do = do.contiguous().to(torch.bfloat16)
            gc, W, U, P, Qg = prepare_cuda(q, k, v, g, beta, scale, True)
            _, _, states = scan_fwd_cuda(q, k, gc, W, U, P, scale, initial_state, True)
            dstates, d_init = scan_bwd_cuda(do, k, gc, W, P, Qg, dfinal)
        else:
            gc, W, U, P, Qg = prepare_reference(q, k, v, g, beta, scale)
            _, _, states = scan_fwd_reference(q, k, gc, W, U, P, scale, initial_state, True)
            dstates, d_init = scan_bwd_reference(do, k, gc, W, P, Qg, dfinal)
        dq, dk, dv, dg, dbeta = chunk_local_grads(q, k, v, g, beta, states, dstates, do, scale)
        if rep > 1:
            dq = dq.reshape(B, T, H // rep, rep, Dk).sum(3)
            dk = dk.reshape(B, T, H // rep, rep, Dk).sum(3)
            q, k = q_in, k_in
        d_init = d_init.reshape(B, H, Dk, Dv).to(initial_state.dtype) if ctx.has_initial else None
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dg.to(g.dtype), dbeta.to(beta.dtype), d_init, None


def gated_delta_rule(q, k, v, g, beta, initial_state=None, scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """q, k ``[B,T,Hk,Dk]``, v ``[B,T,H,Dv]``, g (log decay, <= 0) and beta ``[B,T,H]`` -> (o ``[B,T,H,Dv]``, state ``[B,H,Dk,Dv]``
    fp32).  On a GPU (128-wide heads) q, k, v are taken in bf16 and g, beta in fp32, and ``Hk`` may divide ``H`` (each key head
    serves ``H / Hk`` consecutive value heads without being copied)."""
    scale = float(q.shape[-1] ** -0.5 if scale is None else scale)
    if q.is_cuda:
        q, k, v = (x.to(torch.bfloat16).contiguous() for x in (q, k, v))
        g, beta = g.float().contiguous(), beta.float().contiguous()
    return _GatedDeltaRule.apply(q, k, v, g, beta, initial_state, scale)
