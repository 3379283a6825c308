"""Gated delta net mixer (Qwen3-Next / Qwen3.5 style) and the short causal convolution in front of it.

Parity: src/dew/nn/linear.py:1107-1408 (``GatedDeltaNet``: projections ``in_proj_qkvz`` / ``in_proj_ba``, depthwise causal
``conv1d`` K = 4 + SiLU over [q | k | v], ``A_log``, ``dt_bias``, l2-normalised q and k, ``g = -exp(A_log) softplus(a +
dt_bias)``, ``beta = sigmoid(b)``, chunk-64 scan with fp32 state, gated RMSNorm with ``silu(z)``, ``out_proj``);
src/dew/nn/mixers/gated_delta_net.py (defaults 16 key heads / 32 value heads / 128 / 128 / conv 4); decode paths
src/dew/nn/linear.py:852-1105 (per-row conv window and recurrent state).
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


class ShortConv(nn.Module):
    """Depthwise causal convolution over the sequence axis with optional SiLU; ``weight [C, K]``."""

    def __init__(self, channels: int, kernel_size: int = 4, bias: bool = False, activation: bool = True, dtype=None, device=None):
        super().__init__()
        self.channels, self.kernel_size, self.activation = channels, kernel_size, activation
        self.weight = declare(nn.Parameter(torch.empty(channels, kernel_size, dtype=dtype, device=device)), ("conv", None), "conv_kernel")
        self.bias = declare(nn.Parameter(torch.zeros(channels, dtype=dtype, device=device)), ("conv",), "bias") if bias else None
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            bound = 1.0 / math.sqrt(self.kernel_size)
            self.weight.uniform_(-bound, bound, generator=generator)

    def forward(self, x, segment_ids=None, cache=None):
        if cache is not None and x.shape[1] == 1:
            return scan.short_conv_step(x[:, 0], self.weight, self.bias, cache, self.activation)[:, None]
        y = scan.short_conv(x, self.weight, self.bias, self.activation, segment_ids)
        if cache is not None:
            K = self.kernel_size
            tail = x[:, -(K - 1):]
            cache[:, -tail.shape[1]:] = tail.to(cache.dtype)
        return y


class GatedDeltaNet(nn.Module):
    def __init__(self, features: int, num_k_heads: int = 16, num_v_heads: int = 32, head_k_dim: int = 128, head_v_dim: int = 128,
                 conv_size: int = 4, norm_eps: float = 1e-6, qk_eps: Optional[float] = None, dtype=None, device=None):
        super().__init__()
        self.features = features
        # how q and k are l2-normalised: None - x / max(|x|, 1e-12) (the row kernel on a GPU); a number - x * rsqrt(sum x^2 + qk_eps), the form
        # the Qwen3-Next releases were trained with (1e-6), which differs by a part in a thousand where the projections are small
        self.qk_eps = qk_eps
        self.hk, self.hv, self.dk, self.dv = num_k_heads, num_v_heads, head_k_dim, head_v_dim
        self.key_dim, self.value_dim = num_k_heads * head_k_dim, num_v_heads * head_v_dim
        self.in_proj_qkvz = Linear(features, 2 * self.key_dim + 2 * self.value_dim, axes=("embed", "heads"), dtype=dtype, device=device)
        self.in_proj_ba = Linear(features, 2 * num_v_heads, axes=("embed", "heads"), dtype=dtype, device=device)
        self.conv1d = ShortConv(2 * self.key_dim + self.value_dim, conv_size, activation=True, dtype=dtype, device=device)
        self.A_log = declare(nn.Parameter(torch.zeros(num_v_heads, dtype=torch.float32, device=device)), ("heads",), "A_log")
        self.dt_bias = declare(nn.Parameter(torch.zeros(num_v_heads, dtype=torch.float32, device=device)), ("heads",), "dt_bias")
        self.norm_weight = declare(nn.Parameter(torch.ones(head_v_dim, dtype=dtype, device=device)), ("norm",), "scale")
        self.out_proj = Linear(self.value_dim, features, axes=("heads", "embed"), dtype=dtype, device=device)
        self.norm_eps = norm_eps
        self._own_reset = True
        self.reset_parameters()

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            # A in [1, 16) and dt in [1e-3, 0.1) (log-uniform), the usual state-space initialisation
            dev = self.A_log.device
            if dev.type != "meta":
                a = torch.empty(self.hv, device="cpu").uniform_(1.0, 16.0, generator=None)
                self.A_log.copy_(torch.log(a).to(dev))
                dt = torch.exp(torch.empty(self.hv).uniform_(math.log(1e-3), math.log(0.1)))
                self.dt_bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(dev))
                self.norm_weight.fill_(1.0)

    def forward(self, x, segment_ids=None, cache=None, layer: int = 0):
        B, T, _ = x.shape
        qkvz = self.in_proj_qkvz(x)
        ba = self.in_proj_ba(x).float()
        qkv, z = qkvz[..., : 2 * self.key_dim + self.value_dim], qkvz[..., 2 * self.key_dim + self.value_dim:]
        state = cache.recurrent(layer, B, self) if cache is not None and hasattr(cache, "recurrent") else None
        qkv = self.conv1d(qkv, segment_ids, state["conv"] if state is not None else None)
        q, k, v = qkv.split([self.key_dim, self.key_dim, self.value_dim], -1)
        if self.qk_eps is None:
            q = ops.l2_normalize(q.reshape(B, T, self.hk, self.dk))        # bf16 row kernel on a GPU, fp32 F.normalize elsewhere
            k = ops.l2_normalize(k.reshape(B, T, self.hk, self.dk))
        else:
            q, k = q.reshape(B, T, self.hk, self.dk).float(), k.reshape(B, T, self.hk, self.dk).float()
            q = (q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + self.qk_eps)).to(x.dtype)
            k = (k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + self.qk_eps)).to(x.dtype)
        v = v.reshape(B, T, self.hv, self.dv)
        rep = self.hv // self.hk
        decode = state is not None and T == 1
        if rep > 1 and decode:
            q, k = q.repeat_interleave(rep, 2), k.repeat_interleave(rep, 2)      # the chunked op shares key heads itself
        b, a = ba[..., : self.hv], ba[..., self.hv:]
        beta = torch.sigmoid(b)
        g = -torch.exp(self.A_log.float()) * F.softplus(a + self.dt_bias.float())
        if state is not None and T == 1:
            o = scan.gated_delta_rule_step(q[:, 0], k[:, 0], v[:, 0].float(), g[:, 0], beta[:, 0], state["S"])[:, None]
        else:
            o, S = scan.chunk_gated_delta_rule(q, k, v if v.is_cuda else v.float(), g, beta,
                                               initial_state=state["S"] if state is not None else None)
            if state is not None:
                state["S"].copy_(S)
        o = ops.gated_rms_norm(o.to(x.dtype).reshape(B, T, self.hv, self.dv), z.reshape(B, T, self.hv, self.dv), self.norm_weight, self.norm_eps)
        return self.out_proj(o.reshape(B, T, self.value_dim))


class RecurrentCache:
    """Per-layer decode state of recurrent mixers: the conv window ``[B, K-1, C]`` and the fp32 state ``[B, H, Dk, Dv]``.
    Attention layers of a hybrid stack delegate to the wrapped ``KVStore``."""

    def __init__(self, kv=None):
        self.kv = kv
        self.states = {}

    def recurrent(self, layer: int, batch: int, mixer) -> dict:
        if layer not in self.states:
            p = mixer.out_proj.weight
            if isinstance(mixer, GatedDeltaNet):
                C = 2 * mixer.key_dim + mixer.value_dim
                self.states[layer] = {"conv": torch.zeros(batch, mixer.conv1d.kernel_size - 1, C, dtype=p.dtype, device=p.device),
                                      "S": torch.zeros(batch, mixer.hv, mixer.dk, mixer.dv, dtype=torch.float32, device=p.device)}
            else:
                self.states[layer] = mixer.fresh_state(batch)
        return self.states[layer]

    def attend(self, *args, **kwargs):
        return self.kv.attend(*args, **kwargs)

    def __getattr__(self, name):
        kv = self.__dict__.get("kv")
        if kv is not None and hasattr(kv, name):
            return getattr(kv, name)
        raise AttributeError(name)
