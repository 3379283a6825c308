"""Linear-recurrence ops: gated delta rule (GDN), Mamba-2 SSD, short causal depthwise convolution.

Each op has a step-by-step recurrent form (the fp32 / fp64 oracle and the decode step) and a chunked form
(chunk 64, WY / UT-transform representation for the delta rule) that turns the scan into dense chunk products -
those products are what runs on the tensor cores on a GPU.

Semantics follow the reference: ``S' = (I - beta k k^T) Gamma S + beta k v^T ; o = S'^T q`` with
``g = -exp(A_log) softplus(a + dt_bias)``, ``beta = sigmoid(b)``, l2-normalised q, k, fp32 state
(src/dew/nn/linear.py:1107-1408; src/dew/nn/kernels/recurrence.py:251-329); Mamba-2: decay
``exp(min(acs_i - acs_j, 0))``, fp32 accumulation (src/dew/nn/kernels/mamba_ssd.py:9-22).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

CHUNK_SIZE = 64


# ---------------------------------------------------------------------------------------------------------------
# gated delta rule


def gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=None, scale: Optional[float] = None):
    """Step-by-step oracle. q,k ``[B,T,H,Dk]``, v ``[B,T,H,Dv]``, g / beta ``[B,T,H]`` -> (o ``[B,T,H,Dv]``, state ``[B,H,Dk,Dv]``)."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    dt = torch.float64 if q.dtype == torch.float64 else torch.float32
    scale = scale if scale is not None else Dk ** -0.5
    S = torch.zeros(B, H, Dk, Dv, dtype=dt, device=q.device) if initial_state is None else initial_state.to(dt).clone()
    out = torch.empty(B, T, H, Dv, dtype=dt, device=q.device)
    qf, kf, vf, gf, bf = (x.to(dt) for x in (q, k, v, g, beta))
    for t in range(T):
        S = S * torch.exp(gf[:, t])[..., None, None]
        kt, vt = kf[:, t], vf[:, t]
        pred = torch.einsum("bhkv,bhk->bhv", S, kt)
        S = S + torch.einsum("bhk,bhv->bhkv", kt * bf[:, t][..., None], vt - pred)
        out[:, t] = torch.einsum("bhkv,bhk->bhv", S, qf[:, t] * scale)
    return out.to(v.dtype), S


def gated_delta_rule_step(q, k, v, g, beta, state, scale: Optional[float] = None):
    """One decode step: q,k ``[B,H,Dk]``, v ``[B,H,Dv]``, g / beta ``[B,H]``, state ``[B,H,Dk,Dv]`` (fp32, updated in place)."""
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    state.mul_(torch.exp(g.float())[..., None, None])
    pred = torch.einsum("bhkv,bhk->bhv", state, k.float())
    state.add_(torch.einsum("bhk,bhv->bhkv", k.float() * beta.float()[..., None], v.float() - pred))
    return torch.einsum("bhkv,bhk->bhv", state, q.float() * scale).to(v.dtype)


def gated_delta_rule_chunked(q, k, v, g, beta, initial_state=None, scale: Optional[float] = None, chunk: int = CHUNK_SIZE):
    """Chunked form (WY representation): per chunk, solve ``(I + A) W = beta K`` by forward substitution, then pass the
    state between chunks.  Differentiable; the dense chunk products dominate the cost."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = scale if scale is not None else Dk ** -0.5
    pad = (-T) % chunk
    f32 = torch.float32 if q.dtype != torch.float64 else torch.float64
    qf, kf, vf = (x.to(f32).transpose(1, 2) for x in (q, k, v))              # [B,H,T,D]
    gf, bf = g.to(f32).transpose(1, 2), beta.to(f32).transpose(1, 2)          # [B,H,T]
    if pad:
        qf, kf, vf = (F.pad(x, (0, 0, 0, pad)) for x in (qf, kf, vf))
        gf, bf = F.pad(gf, (0, pad)), F.pad(bf, (0, pad))
    N = (T + pad) // chunk
    qf = qf * scale
    vb = vf * bf[..., None]
    kb = kf * bf[..., None]
    rs = lambda x: x.reshape(B, H, N, chunk, *x.shape[3:])
    qc, kc, vc, kbc, gc = rs(qf), rs(kf), rs(vb), rs(kb), gf.reshape(B, H, N, chunk)
    gc = gc.cumsum(-1)
    diff = gc[..., :, None] - gc[..., None, :]
    tril = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    L = torch.where(tril, torch.exp(torch.where(tril, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    strict = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), -1)
    A = -(kbc @ kc.transpose(-1, -2)) * L
    A = torch.where(strict, A, torch.zeros_like(A))
    # (I - A)^{-1} by forward substitution, row by row (64 small steps; a 16x16-blocked solve on the GPU kernel)
    rows = [A[..., 0, :]]
    for i in range(1, chunk):
        prev = torch.stack(rows, -2)                                           # [..., i, C]
        rows.append(A[..., i, :] + (A[..., i, :i, None] * prev[..., :i, :]).sum(-2))
    Tm = torch.stack(rows, -2) + torch.eye(chunk, dtype=f32, device=q.device)
    U = Tm @ vc                                                                # [B,H,N,C,Dv]
    Wm = Tm @ (kbc * torch.exp(gc)[..., None])                                 # [B,H,N,C,Dk]
    S = torch.zeros(B, H, Dk, Dv, dtype=f32, device=q.device) if initial_state is None else initial_state.to(f32)
    outs = []
    for n in range(N):
        qi, ki, gi = qc[:, :, n], kc[:, :, n], gc[:, :, n]
        attn = torch.where(tril, (qi @ ki.transpose(-1, -2)) * L[:, :, n], torch.zeros_like(L[:, :, n]))
        v_new = U[:, :, n] - Wm[:, :, n] @ S
        o = (qi * torch.exp(gi)[..., None]) @ S + attn @ v_new
        outs.append(o)
        glast = gi[..., -1]
        S = S * torch.exp(glast)[..., None, None] + (ki * torch.exp(glast[..., None] - gi)[..., None]).transpose(-1, -2) @ v_new
    o = torch.stack(outs, 2).reshape(B, H, N * chunk, Dv)[:, :, :T]
    return o.transpose(1, 2).to(v.dtype), S


def chunk_gated_delta_rule(q, k, v, g, beta, initial_state=None, scale=None, chunk: int = CHUNK_SIZE):
    """Public entry.  CUDA tensors with 128-wide keys and values run the sm_100a kernels (``ops/gdn.py``: prepare, forward
    scan, reverse scan on tcgen05); other head sizes on a GPU and every CPU call use the differentiable chunked form."""
    if q.is_cuda and chunk == CHUNK_SIZE:
        from . import gdn
        if gdn.kernel_available(q, v):
            o, S = gdn.gated_delta_rule(q, k, v, g, beta, initial_state, scale)
            return o.to(v.dtype), S
    if q.shape[2] != v.shape[2]:                 # shared key heads: the chunked form works per value head
        rep = v.shape[2] // q.shape[2]
        q, k = q.repeat_interleave(rep, 2), k.repeat_interleave(rep, 2)
    return gated_delta_rule_chunked(q, k, v, g, beta, initial_state, scale, chunk)


# ---------------------------------------------------------------------------------------------------------------
# Mamba-2 SSD


def ssd_recurrent(x, dt, A, Bm, Cm, D=None, initial_state=None):
    """Oracle. x ``[B,T,H,P]``, dt ``[B,T,H]`` (after softplus), A ``[H]`` (negative), B / C ``[B,T,G,N]`` (G groups) ->
    (y ``[B,T,H,P]``, state ``[B,H,P,N]``)."""
    Bsz, T, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    rep = H // G
    f = torch.float64 if x.dtype == torch.float64 else torch.float32
    S = torch.zeros(Bsz, H, P, N, dtype=f, device=x.device) if initial_state is None else initial_state.to(f).clone()
    y = torch.empty(Bsz, T, H, P, dtype=f, device=x.device)
    xf, dtf, Bf, Cf = x.to(f), dt.to(f), Bm.to(f).repeat_interleave(rep, 2), Cm.to(f).repeat_interleave(rep, 2)
    for t in range(T):
        dA = torch.exp(dtf[:, t] * A.to(f))                                   # [B,H]
        S = S * dA[..., None, None] + torch.einsum("bhp,bhn->bhpn", xf[:, t] * dtf[:, t][..., None], Bf[:, t])
        y[:, t] = torch.einsum("bhpn,bhn->bhp", S, Cf[:, t])
    if D is not None:
        y = y + xf * D.to(f)[None, None, :, None]
    return y.to(x.dtype), S


def ssd(x, dt, A, Bm, Cm, D=None, initial_state=None):
    """Public entry: CUDA tensors with head dimension 64 and state dimension 128 run the sm_100a scan kernel
    (``ops/ssd.py``); everything else the loop-free chunked form below."""
    if x.is_cuda:
        from . import ssd as K
        if K.kernel_available(x, Bm):
            return K.ssd(x, dt, A, Bm, Cm, D, initial_state)
    return ssd_chunked(x, dt, A, Bm, Cm, D, initial_state)


def ssd_chunked(x, dt, A, Bm, Cm, D=None, initial_state=None, chunk: int = CHUNK_SIZE):
    """Chunked SSD: intra-chunk ``(C B^T o decay) X`` plus a chunk-state pass; fp32 accumulation."""
    Bsz, T, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    rep = H // G
    f = torch.float32 if x.dtype != torch.float64 else torch.float64
    pad = (-T) % chunk
    xf, dtf = x.to(f), dt.to(f)
    Bf, Cf = Bm.to(f).repeat_interleave(rep, 2), Cm.to(f).repeat_interleave(rep, 2)
    if pad:
        xf, Bf, Cf = (F.pad(t_, (0, 0, 0, 0, 0, pad)) for t_ in (xf, Bf, Cf))
        dtf = F.pad(dtf, (0, 0, 0, pad))
    Nc = (T + pad) // chunk
    rs = lambda t_: t_.reshape(Bsz, Nc, chunk, *t_.shape[2:])
    xc, Bc, Cc, dtc = rs(xf), rs(Bf), rs(Cf), rs(dtf)                          # [B,Nc,C,H,...]
    a = dtc * A.to(f)                                                          # [B,Nc,C,H] log decay per step
    acs = a.cumsum(2)
    diff = acs[:, :, :, None, :] - acs[:, :, None, :, :]                       # [B,Nc,C(i),C(j),H]
    tril = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=x.device))[None, None, :, :, None]
    Lm = torch.where(tril, torch.exp(torch.clamp(diff, max=0.0)), torch.zeros_like(diff))
    xdt = xc * dtc[..., None]
    CB = torch.einsum("bcihn,bcjhn->bcijh", Cc, Bc)
    y_diag = torch.einsum("bcijh,bcjhp->bcihp", CB * Lm, xdt)
    decay_to_end = torch.exp(acs[:, :, -1:, :] - acs)                          # [B,Nc,C,H]
    states = torch.einsum("bcjhn,bcjh,bcjhp->bchpn", Bc, decay_to_end, xdt)    # contribution of each chunk
    S0 = torch.zeros(Bsz, H, P, N, dtype=f, device=x.device) if initial_state is None else initial_state.to(f)
    # state passing without a loop over chunks: the state on entry to chunk c is sum_{c' < c} exp(sum of the chunk decays
    # between them) * (chunk c' contribution), one [Nc + 1, Nc + 1] lower-triangular product per (batch, head)
    tot = acs[:, :, -1, :]                                                      # [B,Nc,H] log decay of each whole chunk
    csum = torch.cat([torch.zeros_like(tot[:, :1]), tot.cumsum(1)], 1)         # [B,Nc+1,H]
    seg = csum[:, :, None, :] - csum[:, None, :, :]                            # [B, c, c', H]: decay from the end of chunk c'-1 ... to the start of chunk c
    lower = torch.tril(torch.ones(Nc + 1, Nc + 1, dtype=torch.bool, device=x.device), -1)[None, :, :, None]
    contrib = torch.cat([S0[:, None], states], 1)                              # entry 0: the initial state, entry c'+1: chunk c'
    # state before chunk c = sum_{e <= c} exp(csum[c] - csum[e]) * contrib[e]
    le = torch.tril(torch.ones(Nc + 1, Nc + 1, dtype=torch.bool, device=x.device))[None, :, :, None]
    wts = torch.where(le, torch.exp(torch.where(le, seg, torch.zeros_like(seg))), torch.zeros_like(seg))
    entry = torch.einsum("bceh,behpn->bchpn", wts, contrib)                     # [B,Nc+1,H,P,N]; entry[c] = state before chunk c
    del lower
    y_off = torch.einsum("bcihn,bchpn,bcih->bcihp", Cc, entry[:, :Nc], torch.exp(acs))
    y = (y_diag + y_off).reshape(Bsz, Nc * chunk, H, P)[:, :T]
    S = entry[:, Nc]
    if D is not None:
        y = y + x.to(f) * D.to(f)[None, None, :, None]
    return y.to(x.dtype), S


def ssd_step(x, dt, A, Bm, Cm, state, D=None):
    """One decode step: x ``[B,H,P]``, dt ``[B,H]``, B / C ``[B,G,N]``; ``state [B,H,P,N]`` fp32 updated in place."""
    H, G = x.shape[1], Bm.shape[1]
    Bf, Cf = Bm.float().repeat_interleave(H // G, 1), Cm.float().repeat_interleave(H // G, 1)
    state.mul_(torch.exp(dt.float() * A.float())[..., None, None])
    state.add_(torch.einsum("bhp,bhn->bhpn", x.float() * dt.float()[..., None], Bf))
    y = torch.einsum("bhpn,bhn->bhp", state, Cf)
    if D is not None:
        y = y + x.float() * D.float()[None, :, None]
    return y.to(x.dtype)


# ---------------------------------------------------------------------------------------------------------------
# short causal depthwise convolution


def short_conv_reference(x, w, bias=None, activation: bool = True, segment_ids=None, initial=None):
    """``y[t] = act(sum_j w[c, j] x[t - K + 1 + j] + b)``; x ``[B,T,C]``, w ``[C,K]``.  With ``segment_ids [B,T]`` taps
    that would cross a document boundary are dropped (packed documents).  ``initial [B,K-1,C]`` prepends history."""
    B, T, C = x.shape
    K = w.shape[1]
    xf = x.float()
    hist = torch.zeros(B, K - 1, C, dtype=torch.float32, device=x.device) if initial is None else initial.float()
    xp = torch.cat([hist, xf], 1)
    y = torch.zeros(B, T, C, dtype=torch.float32, device=x.device)
    for j in range(K):
        tap = xp[:, j:j + T]
        if segment_ids is not None:
            shift = K - 1 - j
            if shift > 0:
                same = torch.ones(B, T, dtype=torch.bool, device=x.device)
                same[:, shift:] = segment_ids[:, shift:] == segment_ids[:, :-shift]
                same[:, :shift] = initial is not None
                tap = tap * same[..., None]
        y = y + tap * w[:, j].float()
    if bias is not None:
        y = y + bias.float()
    if activation:
        y = F.silu(y)
    return y.to(x.dtype)


def short_conv(x, w, bias=None, activation: bool = True, segment_ids=None, initial=None):
    from . import library as L
    if L.use_cuda(x) and x.dtype == torch.bfloat16 and segment_ids is None and initial is None and hasattr(L.load(), "dewb_short_conv_fwd") \
            and x.shape[-1] % 8 == 0 and 2 <= w.shape[1] <= 4:
        from .conv import short_conv_cuda
        return short_conv_cuda(x, w, bias, activation)
    return short_conv_reference(x, w, bias, activation, segment_ids, initial)


def short_conv_step(x, w, bias, cache, activation: bool = True):
    """Decode step: x ``[B,C]``; ``cache [B,K-1,C]`` holds the last K-1 inputs and is rolled in place."""
    K = w.shape[1]
    window = torch.cat([cache, x[:, None].to(cache.dtype)], 1)                 # [B,K,C]
    y = (window.float() * w.float().t()[None]).sum(1)
    if bias is not None:
        y = y + bias.float()
    cache.copy_(window[:, 1:])
    return (F.silu(y) if activation else y).to(x.dtype)


# ---------------------------------------------------------------------------------------------------------------
# Kimi delta attention (KDA): the gated delta rule with a per-channel (not per-head) decay.
# Reference: src/dew/nn/kernels/fla_kda.py (chunked kernels), src/dew/nn/kda.py.
def kda_recurrent(q, k, v, g, beta, initial_state=None, scale: Optional[float] = None):
    """``q, k [B,T,H,Dk]``, ``v [B,T,H,Dv]``, ``g [B,T,H,Dk]`` (log decay per key channel, <= 0), ``beta [B,T,H]``.
    ``S_t = (I - beta k k^T) diag(exp(g_t)) S_{t-1} + beta k v^T``;  ``o_t = S_t^T q_t * scale``.  fp32 state."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = Dk ** -0.5 if scale is None else scale
    S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=q.device) if initial_state is None else initial_state.float().clone()
    out = []
    qf, kf, vf, gf, bf = q.float(), k.float(), v.float(), g.float(), beta.float()
    for t in range(T):
        S = S * gf[:, t].exp().unsqueeze(-1)
        kv = torch.einsum("bhk,bhkv->bhv", kf[:, t], S)
        S = S + torch.einsum("bhk,bhv->bhkv", kf[:, t], (vf[:, t] - kv) * bf[:, t].unsqueeze(-1))
        out.append(torch.einsum("bhk,bhkv->bhv", qf[:, t] * scale, S))
    return torch.stack(out, 1).to(v.dtype), S


def kda_chunked(q, k, v, g, beta, initial_state=None, scale: Optional[float] = None, chunk: int = CHUNK_SIZE):
    """Chunk-parallel form: inside a chunk the decay is folded into q and k (``q~ = q exp(G)``, ``k~ = k exp(-G)`` with
    ``G`` the running sum of ``g``), which reduces the recurrence to the ungated delta rule's WY representation; the state
    crosses chunks in fp32.  Equals ``kda_recurrent`` up to rounding."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = Dk ** -0.5 if scale is None else scale
    pad = (-T) % chunk
    if pad:
        z = lambda x: torch.nn.functional.pad(x, (0, 0) * (x.dim() - 2) + (0, pad))
        q, k, v, g = z(q), z(k), z(v), z(g)
        beta = torch.nn.functional.pad(beta, (0, 0, 0, pad))
    N = q.shape[1] // chunk
    f = lambda x: x.float().reshape(B, N, chunk, H, -1).permute(0, 1, 3, 2, 4)          # [B,N,H,C,D]
    qf, kf, vf, gf = f(q) * scale, f(k), f(v), f(g)
    bf = beta.float().reshape(B, N, chunk, H).permute(0, 1, 3, 2)                       # [B,N,H,C]
    G = gf.cumsum(-2)                                                                   # [B,N,H,C,Dk]
    qd, kd = qf * G.exp(), kf * (-G).exp()                                              # decay folded in
    kb = kf * G.exp()                                                                   # key as the state of chunk start sees it
    S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=q.device) if initial_state is None else initial_state.float().clone()
    eye = torch.eye(chunk, device=q.device)
    lower = torch.tril(torch.ones(chunk, chunk, device=q.device), -1)
    outs = []
    for n in range(N):
        A = torch.einsum("bhik,bhjk->bhij", kb[:, n], kd[:, n]) * lower * bf[:, n].unsqueeze(-1)      # strictly lower
        Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)        # (I + A)^-1
        rhs = (vf[:, n] - torch.einsum("bhik,bhkv->bhiv", kb[:, n], S)) * bf[:, n].unsqueeze(-1)
        U = torch.einsum("bhij,bhjv->bhiv", Tm, rhs)                                    # corrected values
        attn = torch.einsum("bhik,bhjk->bhij", qd[:, n], kd[:, n]) * (lower + eye)
        outs.append(torch.einsum("bhik,bhkv->bhiv", qd[:, n], S) + torch.einsum("bhij,bhjv->bhiv", attn, U))
        last = G[:, n, :, -1]                                                           # [B,H,Dk]
        S = S * last.exp().unsqueeze(-1) + torch.einsum("bhik,bhiv->bhkv", kd[:, n] * last.exp().unsqueeze(-2), U)
    o = torch.stack(outs, 1).permute(0, 1, 3, 2, 4).reshape(B, N * chunk, H, Dv)[:, :T]
    return o.to(v.dtype), S


# ---------------------------------------------------------------------------------------------------------------
# Mamba-1 selective scan.  Reference: src/dew/nn/kernels/templates/recurrence/selective.py, src/dew/nn/mixers/mamba.py.
def selective_scan_reference(x, dt, A, Bm, Cm, D=None, z=None, initial_state=None):
    """``x, dt [B,T,C]``, ``A [C,N]`` (negative), ``Bm, Cm [B,T,N]``: ``h_t = exp(dt A) h_{t-1} + dt B x``; ``y = C h + D x``,
    optionally gated by ``silu(z)``.  Sequential over T, fp32 state ``[B,C,N]``."""
    Bsz, T, C = x.shape
    h = torch.zeros(Bsz, C, A.shape[1], dtype=torch.float32, device=x.device) if initial_state is None else initial_state.float().clone()
    xf, dtf, Af, Bf, Cf = x.float(), dt.float(), A.float(), Bm.float(), Cm.float()
    ys = []
    for t in range(T):
        dA = torch.exp(dtf[:, t].unsqueeze(-1) * Af)
        h = dA * h + (dtf[:, t] * xf[:, t]).unsqueeze(-1) * Bf[:, t].unsqueeze(1)
        ys.append(torch.einsum("bcn,bn->bc", h, Cf[:, t]))
    y = torch.stack(ys, 1)
    if D is not None:
        y = y + xf * D.float()
    if z is not None:
        y = y * torch.nn.functional.silu(z.float())
    return y.to(x.dtype), h


def selective_scan(x, dt, A, Bm, Cm, D=None, z=None, initial_state=None, chunk: int = 64):
    """Chunked selective scan: a log-depth (Hillis-Steele) prefix combine of ``(decay, increment)`` pairs inside each chunk,
    state carried across chunks - O(T log chunk) parallel work instead of T sequential steps."""
    Bsz, T, C = x.shape
    N = A.shape[1]
    pad = (-T) % chunk
    xf, dtf = x.float(), dt.float()
    Bf, Cf = Bm.float(), Cm.float()
    if pad:
        p3 = lambda t: torch.nn.functional.pad(t, (0, 0, 0, pad))
        xf, dtf, Bf, Cf = p3(xf), p3(dtf), p3(Bf), p3(Cf)
    n = xf.shape[1] // chunk
    a = torch.exp(dtf.unsqueeze(-1) * A.float()).reshape(Bsz, n, chunk, C, N)                      # decay per step
    b = ((dtf * xf).unsqueeze(-1) * Bf.unsqueeze(2)).reshape(Bsz, n, chunk, C, N)                  # increment per step
    # inclusive scan of the affine maps h -> a h + b along the chunk axis
    step = 1
    while step < chunk:
        a_prev = torch.cat([torch.ones_like(a[:, :, :step]), a[:, :, :-step]], 2)
        b_prev = torch.cat([torch.zeros_like(b[:, :, :step]), b[:, :, :-step]], 2)
        b = a * b_prev + b
        a = a * a_prev
        step *= 2
    h = torch.zeros(Bsz, C, N, dtype=torch.float32, device=x.device) if initial_state is None else initial_state.float().clone()
    ys = []
    Cc = Cf.reshape(Bsz, n, chunk, N)
    for i in range(n):
        hs = a[:, i] * h.unsqueeze(1) + b[:, i]                                                   # [B, chunk, C, N]
        ys.append(torch.einsum("btcn,btn->btc", hs, Cc[:, i]))
        h = hs[:, -1]
    y = torch.cat(ys, 1)[:, :T]
    if D is not None:
        y = y + x.float() * D.float()
    if z is not None:
        y = y * torch.nn.functional.silu(z.float())
    return y.to(x.dtype), h


# ---------------------------------------------------------------------------------------------------------------
# RWKV-4 time mixing (wkv).  Reference: src/dew/nn/kernels/wkv4.py.
def wkv4(w, u, k, v):
    """``w, u [C]`` (decay ``exp(-exp(w))`` per channel, bonus ``u``), ``k, v [B,T,C]``: the numerically stable running
    ratio ``(sum_j<t e^{-(t-1-j) e^w + k_j} v_j + e^{u + k_t} v_t) / (same with v = 1)``."""
    B, T, C = k.shape
    wf, uf, kf, vf = -torch.exp(w.float()), u.float(), k.float(), v.float()
    num = torch.zeros(B, C, device=k.device); den = torch.zeros(B, C, device=k.device)
    mx = torch.full((B, C), -1e38, device=k.device)
    out = []
    for t in range(T):
        kt, vt = kf[:, t], vf[:, t]
        m1 = torch.maximum(mx, uf + kt)
        e1, e2 = torch.exp(mx - m1), torch.exp(uf + kt - m1)
        out.append((e1 * num + e2 * vt) / (e1 * den + e2))
        m2 = torch.maximum(mx + wf, kt)
        e1, e2 = torch.exp(mx + wf - m2), torch.exp(kt - m2)
        num, den, mx = e1 * num + e2 * vt, e1 * den + e2, m2
    return torch.stack(out, 1).to(v.dtype)
