"""Mamba-2 mixer: input projection to ``[z | x | B | C | dt]``, short causal conv over ``[x | B | C]``, chunked SSD scan,
gated RMSNorm, output projection.

Parity: src/dew/nn/mixers/mamba2.py:101-587 (``chunk_ssd`` :101, ``recurrent_ssd`` :139, ``MambaRMSNormGated`` :194,
``Mamba2`` :233), numerics src/dew/nn/kernels/mamba_ssd.py:9-22.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import scan
from .layers import Linear, declare
from .linear_attention import ShortConv


class Mamba2(nn.Module):
    def __init__(self, features: int, state_dim: int = 128, head_dim: int = 64, expand: int = 2, groups: int = 1, conv_size: int = 4,
                 norm_eps: float = 1e-6, gate_after: bool = False, dtype=None, device=None):
        super().__init__()
        self.gate_after = gate_after
        self.features, self.N, self.P, self.G = features, state_dim, head_dim, groups
        self.inner = expand * features
        self.H = self.inner // head_dim
        self.in_proj = Linear(features, 2 * self.inner + 2 * groups * state_dim + self.H, axes=("embed", "mlp"), dtype=dtype, device=device)
        self.conv1d = ShortConv(self.inner + 2 * groups * state_dim, conv_size, bias=True, dtype=dtype, device=device)
        self.A_log = declare(nn.Parameter(torch.zeros(self.H, dtype=torch.float32, device=device)), ("heads",), "A_log")
        self.dt_bias = declare(nn.Parameter(torch.zeros(self.H, dtype=torch.float32, device=device)), ("heads",), "dt_bias")
        self.D = declare(nn.Parameter(torch.ones(self.H, dtype=torch.float32, device=device)), ("heads",), "scale")
        self.norm_weight = declare(nn.Parameter(torch.ones(self.inner, dtype=dtype, device=device)), ("norm",), "scale")
        self.out_proj = Linear(self.inner, features, axes=("mlp", "embed"), dtype=dtype, device=device)
        self.norm_eps = norm_eps
        self._own_reset = True
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            if self.A_log.device.type != "meta":
                self.A_log.copy_(torch.log(torch.empty(self.H).uniform_(1.0, 16.0)).to(self.A_log.device))
                dt = torch.exp(torch.empty(self.H).uniform_(math.log(1e-3), math.log(0.1)))
                self.dt_bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(self.dt_bias.device))
                self.D.fill_(1.0)
                self.norm_weight.fill_(1.0)

    def fresh_state(self, batch: int) -> dict:
        p = self.out_proj.weight
        C = self.inner + 2 * self.G * self.N
        return {"conv": torch.zeros(batch, self.conv1d.kernel_size - 1, C, dtype=p.dtype, device=p.device),
                "S": torch.zeros(batch, self.H, self.P, self.N, dtype=torch.float32, device=p.device)}

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0):
        B, T, _ = x.shape
        zxbcdt = self.in_proj(x)
        z, xbc, dt = zxbcdt.split([self.inner, self.inner + 2 * self.G * self.N, self.H], -1)
        state = cache.recurrent(layer, B, self) if cache is not None and hasattr(cache, "recurrent") else None
        xbc = self.conv1d(xbc, segment_ids, state["conv"] if state is not None else None)
        xs, Bm, Cm = xbc.split([self.inner, self.G * self.N, self.G * self.N], -1)
        dt = F.softplus(dt.float() + self.dt_bias.float())
        A = -torch.exp(self.A_log.float())
        xs = xs.reshape(B, T, self.H, self.P)
        Bm, Cm = Bm.reshape(B, T, self.G, self.N), Cm.reshape(B, T, self.G, self.N)
        if state is not None and T == 1:
            y = scan.ssd_step(xs[:, 0], dt[:, 0], A, Bm[:, 0], Cm[:, 0], state["S"], self.D)[:, None]
        else:
            y, S = scan.ssd(xs, dt, A, Bm, Cm, self.D, initial_state=state["S"] if state is not None else None)
            if state is not None:
                state["S"].copy_(S)
        y = y.to(x.dtype).reshape(B, T, self.inner)
        if self.gate_after:
            y = ops.gated_rms_norm(y, z, self.norm_weight, self.norm_eps)              # norm, then gate (Falcon-H1's order)
        else:
            # Mamba-2's own order: the gate first, the norm over the whole width after (modeling_mamba2.py MambaRMSNormGated)
            y = ops.rms_norm((y.float() * F.silu(z.float())).to(x.dtype), self.norm_weight, self.norm_eps)
        return self.out_proj(y)
