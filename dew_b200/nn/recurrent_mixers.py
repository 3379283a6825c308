"""More recurrent mixers: lightning attention (MiniMax), the S5 diagonal state space layer, and Mamba-3's single-input
single-output recurrence (exponential-trapezoidal discretisation, complex state).

Each has the step-by-step recurrence as its oracle and a parallel form that is what training runs:
* lightning attention is the SSD recurrence with a constant decay per head (``dt = 1``, ``A = -rate``), so on a GPU with
  64-wide heads and 128-wide keys it runs the SSD scan kernel (``ops.scan.ssd``);
* S5 runs its diagonal complex recurrence as a log-depth scan of affine maps;
* Mamba-3 folds the state's rotation into B and C (cumulative angles) and the previous token's write into each token's
  own weight, which turns it into a decayed linear attention evaluated chunk by chunk.

Reference: src/dew/nn/mixers/lightning.py (``S_t = e^{-r} S_{t-1} + k_t v_t^T``, ALiBi-slope rates scaled by depth, RMS norm
over all heads, sigmoid output gate), src/dew/nn/ssm.py (S5 from the S4D-Lin poles), src/dew/nn/mixers/mamba3.py
(``h_t = e^{-i dt theta}(alpha h_{t-1} + beta B_{t-1} x_{t-1}) + gamma B_t x_t``, ``y_t = Re(C_t^* h_t)``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import scan
from .layers import Linear, declare


# ---------------------------------------------------------------------------------------------------------------
# lightning attention


def alibi_slopes(heads: int) -> torch.Tensor:
    """ALiBi's geometric slopes for ``heads`` heads (closest power of two, then the interleaved remainder)."""
    def power_of_two(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start * start ** i for i in range(n)]
    if math.log2(heads).is_integer():
        return torch.tensor(power_of_two(heads))
    base = 2 ** math.floor(math.log2(heads))
    return torch.tensor(power_of_two(base) + power_of_two(2 * base)[0::2][: heads - base])


def lightning_recurrent(q, k, v, rate, state=None):
    """Oracle. q, k ``[B,T,H,Dk]``, v ``[B,T,H,Dv]``, rate ``[H]`` (>= 0) -> (o ``[B,T,H,Dv]``, state ``[B,H,Dk,Dv]``)."""
    B, T, H, Dk = q.shape
    f = torch.float64 if q.dtype == torch.float64 else torch.float32
    S = torch.zeros(B, H, Dk, v.shape[-1], dtype=f, device=q.device) if state is None else state.to(f).clone()
    decay = torch.exp(-rate.to(f))[None, :, None, None]
    out = []
    for t in range(T):
        S = S * decay + torch.einsum("bhk,bhv->bhkv", k[:, t].to(f), v[:, t].to(f))
        out.append(torch.einsum("bhk,bhkv->bhv", q[:, t].to(f), S))
    return torch.stack(out, 1).to(v.dtype), S


def lightning_attention(q, k, v, rate, state=None):
    """The same through the SSD scan (x = v, B = k, C = q, dt = 1, A = -rate): kernel on a GPU, chunked form elsewhere.
    The SSD state is ``[B,H,Dv,Dk]``; it is returned transposed to the recurrence's ``[B,H,Dk,Dv]``."""
    B, T, H, _ = q.shape
    dt = torch.ones(B, T, H, dtype=torch.float32, device=q.device)
    init = None if state is None else state.transpose(-1, -2)
    y, S = scan.ssd(v, dt, -rate.float(), k, q, None, init)
    return y, S.transpose(-1, -2)


class LightningAttention(nn.Module):
    def __init__(self, features: int, num_heads: int = 8, head_dim: int = 64, depth: int = 0, layers: int = 1, norm_eps: float = 1e-6,
                 dtype=None, device=None):
        super().__init__()
        self.h, self.d = num_heads, head_dim
        inner = num_heads * head_dim
        self.qkv = Linear(features, 3 * inner, axes=("embed", "heads"), dtype=dtype, device=device)
        self.output_gate = Linear(features, inner, axes=("embed", "heads"), dtype=dtype, device=device)
        self.norm_weight = declare(nn.Parameter(torch.ones(inner, dtype=dtype, device=device)), ("norm",), "scale")
        self.out_proj = Linear(inner, features, axes=("heads", "embed"), dtype=dtype, device=device)
        self.eps = norm_eps
        # the first layer forgets fastest: slope * (1 - depth / (layers - 1) + 1e-5)
        factor = 1.0 - depth / max(layers - 1, 1) + 1e-5
        self.register_buffer("rate", alibi_slopes(num_heads).float() * factor, persistent=False)

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0):
        B, T, _ = x.shape
        q, k, v = F.silu(self.qkv(x)).view(B, T, 3, self.h, self.d).unbind(2)
        state = cache.recurrent(layer, B, self) if cache is not None and hasattr(cache, "recurrent") else None
        o, S = lightning_attention(q, k, v, self.rate.to(x.device), state["S"] if state is not None else None)
        if state is not None:
            state["S"].copy_(S)
        o = ops.rms_norm(o.reshape(B, T, -1).to(x.dtype), self.norm_weight, self.eps)
        return self.out_proj(o * torch.sigmoid(self.output_gate(x)))

    def fresh_state(self, batch: int) -> dict:
        p = self.out_proj.weight
        return {"S": torch.zeros(batch, self.h, self.d, self.d, dtype=torch.float32, device=p.device)}


# ---------------------------------------------------------------------------------------------------------------
# S5


def affine_scan(a: torch.Tensor, b: torch.Tensor, dim: int = 1):
    """Inclusive scan of ``h_t = a_t h_{t-1} + b_t`` (h_{-1} = 0) along ``dim`` in log2(T) doubling steps (real or complex)."""
    T = a.shape[dim]
    step = 1
    a, b = a.clone(), b.clone()
    while step < T:
        idx_hi = torch.arange(step, T, device=a.device)
        a_prev, b_prev = a.index_select(dim, idx_hi - step), b.index_select(dim, idx_hi - step)
        a_hi, b_hi = a.index_select(dim, idx_hi), b.index_select(dim, idx_hi)
        b = b.index_copy(dim, idx_hi, a_hi * b_prev + b_hi)
        a = a.index_copy(dim, idx_hi, a_hi * a_prev)
        step *= 2
    return b


class S5Layer(nn.Module):
    """Diagonal complex state space layer: ``h_t = Lambda_bar h_{t-1} + B_bar u_t``, ``y_t = Re(C h_t) + D u_t`` with the
    S4D-Lin poles ``Lambda_n = -1/2 + i pi n`` and a learned per-state step size (zero-order hold)."""

    def __init__(self, features: int, state_dim: int = 64, dt_min: float = 1e-3, dt_max: float = 1e-1, dtype=None, device=None):
        super().__init__()
        self.features, self.n = features, state_dim
        n = torch.arange(state_dim, dtype=torch.float32, device=device)
        self.lambda_re = nn.Parameter(torch.full((state_dim,), -0.5, device=device))
        self.lambda_im = nn.Parameter(math.pi * n)
        self.B = nn.Parameter(torch.randn(state_dim, features, 2, device=device) / math.sqrt(2 * features))
        self.C = nn.Parameter(torch.randn(features, state_dim, 2, device=device) / math.sqrt(state_dim))
        self.D = nn.Parameter(torch.ones(features, device=device))
        self.log_dt = nn.Parameter(torch.empty(state_dim, device=device).uniform_(math.log(dt_min), math.log(dt_max)))

    def discretised(self):
        lam = torch.complex(self.lambda_re.clamp(max=-1e-4), self.lambda_im)        # poles stay in the left half plane
        dt = torch.exp(self.log_dt)
        lam_bar = torch.exp(lam * dt)
        b_bar = ((lam_bar - 1) / lam)[:, None] * torch.view_as_complex(self.B)
        return lam_bar, b_bar, torch.view_as_complex(self.C)

    def forward(self, u: torch.Tensor, recurrent: bool = False) -> torch.Tensor:
        """``u [B,T,features] -> [B,T,features]``."""
        lam_bar, b_bar, c = self.discretised()
        bu = torch.einsum("nf,btf->btn", b_bar, u.float().to(b_bar.dtype))
        if recurrent:
            h = torch.zeros(u.shape[0], self.n, dtype=bu.dtype, device=u.device)
            hs = []
            for t in range(u.shape[1]):
                h = lam_bar * h + bu[:, t]
                hs.append(h)
            hs = torch.stack(hs, 1)
        else:
            hs = affine_scan(lam_bar.expand_as(bu), bu, 1)
        y = torch.einsum("fn,btn->btf", c, hs).real + u.float() * self.D
        return y.to(u.dtype)


# ---------------------------------------------------------------------------------------------------------------
# Mamba-3 (single input, single output)


def mamba3_recurrent(x, dt, A, Bm, Cm, theta, lam):
    """Oracle on the complex state.  x ``[B,T,H,P]``; dt, lam ``[B,T,H]``; A ``[H]`` (negative); Bm, Cm ``[B,T,H,N]`` (N even: pairs
    ``(2j, 2j+1)`` are the complex numbers ``v_2j + i v_2j+1``); theta ``[B,T,H,N/2]``.
    ``h_t = e^{-i dt theta}(alpha h_{t-1} + beta B_{t-1} x_{t-1}) + gamma B_t x_t``; ``y_t = Re(C_t^* h_t)`` with
    ``alpha = e^{dt A}``, ``beta = (1 - lam) dt alpha``, ``gamma = lam dt``."""
    Bsz, T, H, P = x.shape
    f = torch.float64 if x.dtype == torch.float64 else torch.float32
    cplx = lambda v: torch.view_as_complex(v.to(f).reshape(*v.shape[:-1], v.shape[-1] // 2, 2).contiguous())
    Bc, Cc = cplx(Bm), cplx(Cm)
    h = torch.zeros(Bsz, H, P, Bc.shape[-1], dtype=Bc.dtype, device=x.device)
    prev = torch.zeros_like(h)
    ys = []
    for t in range(T):
        alpha = torch.exp(dt[:, t].to(f) * A.to(f))
        beta = (1 - lam[:, t].to(f)) * dt[:, t].to(f) * alpha
        gamma = lam[:, t].to(f) * dt[:, t].to(f)
        turn = torch.exp(torch.complex(torch.zeros_like(theta[:, t].to(f)), -(dt[:, t].to(f)[..., None] * theta[:, t].to(f))))
        write = torch.einsum("bhp,bhn->bhpn", x[:, t].to(f).to(Bc.dtype), Bc[:, t])
        h = turn[:, :, None] * (alpha[..., None, None] * h + beta[..., None, None] * prev) + gamma[..., None, None] * write
        prev = write
        ys.append(torch.einsum("bhn,bhpn->bhp", Cc[:, t].conj(), h).real)
    return torch.stack(ys, 1).to(x.dtype)


def mamba3_parallel(x, dt, A, Bm, Cm, theta, lam):
    """The same as a decayed linear attention: with ``phi_t = sum_{s <= t} dt_s theta_s`` (cumulative angle) and
    ``g_t = sum_{s <= t} dt_s A``, token u's value reaches token t >= u at weight
    ``w_u(t) e^{g_t - g_u} Re(conj(C_t e^{i phi_t})^* ... )``: B and C are turned by their own angles, the previous token's write is
    folded into the token's own at weight ``delta_{u+1} = (1 - lam_{u+1}) dt_{u+1}`` for every later reader and ``gamma_u`` alone
    for the token itself."""
    Bsz, T, H, P = x.shape
    f = torch.float64 if x.dtype == torch.float64 else torch.float32
    cplx = lambda v: torch.view_as_complex(v.to(f).reshape(*v.shape[:-1], v.shape[-1] // 2, 2).contiguous())
    dtf, lamf = dt.to(f), lam.to(f)
    phi = (dtf[..., None] * theta.to(f)).cumsum(1)                                   # [B,T,H,N/2]
    rot = torch.exp(torch.complex(torch.zeros_like(phi), phi))
    Bt, Ct = cplx(Bm) * rot, cplx(Cm) * rot                                         # turned keys and queries
    g = (dtf * A.to(f)).cumsum(1)                                                    # [B,T,H]
    gamma = lamf * dtf
    delta_next = torch.cat([((1 - lamf) * dtf)[:, 1:], torch.zeros_like(dtf[:, :1])], 1)
    scores = torch.einsum("bthn,buhn->bhtu", Ct.conj(), Bt).real                     # Re(C_t^* B_u) after the turns
    decay = torch.exp((g.permute(0, 2, 1)[..., :, None] - g.permute(0, 2, 1)[..., None, :]).clamp(max=0.0))
    strict = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device), -1)
    w_later = (gamma + delta_next).permute(0, 2, 1)[..., None, :]                    # weight of u for every later t
    w_own = gamma.permute(0, 2, 1)
    attn = torch.where(strict, scores * decay * w_later, torch.zeros_like(scores))
    attn = attn + torch.diag_embed(torch.diagonal(scores, dim1=-2, dim2=-1) * w_own)
    return torch.einsum("bhtu,buhp->bthp", attn, x.to(f)).to(x.dtype)


class Mamba3(nn.Module):
    def __init__(self, features: int, state_dim: int = 64, head_dim: int = 64, expand: int = 2, norm_eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.N, self.P = state_dim, head_dim
        self.inner = expand * features
        self.H = self.inner // head_dim
        H, N = self.H, self.N
        self.in_proj = Linear(features, 2 * self.inner + 2 * H * N + H * (N // 2) + 2 * H, axes=("embed", "mlp"), dtype=dtype, device=device)
        self.A_log = declare(nn.Parameter(torch.log(torch.empty(H, device=device).uniform_(1.0, 16.0))), ("heads",), "A_log")
        self.dt_bias = declare(nn.Parameter(torch.zeros(H, dtype=torch.float32, device=device)), ("heads",), "dt_bias")
        self.norm_weight = declare(nn.Parameter(torch.ones(self.inner, dtype=dtype, device=device)), ("norm",), "scale")
        self.out_proj = Linear(self.inner, features, axes=("mlp", "embed"), dtype=dtype, device=device)
        self.eps = norm_eps

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0, recurrent: bool = False):
        B, T, _ = x.shape
        H, N, P = self.H, self.N, self.P
        z, xs, Bm, Cm, theta, dt, lam = self.in_proj(x).split([self.inner, self.inner, H * N, H * N, H * (N // 2), H, H], -1)
        dt = F.softplus(dt.float() + self.dt_bias)
        lam = torch.sigmoid(lam.float())
        A = -torch.exp(self.A_log.float())
        fn = mamba3_recurrent if recurrent else mamba3_parallel
        y = fn(xs.reshape(B, T, H, P).float(), dt, A, Bm.reshape(B, T, H, N).float(), Cm.reshape(B, T, H, N).float(),
               theta.reshape(B, T, H, N // 2).float(), lam)
        y = ops.gated_rms_norm(y.reshape(B, T, self.inner).to(x.dtype), z, self.norm_weight, self.eps)
        return self.out_proj(y)
