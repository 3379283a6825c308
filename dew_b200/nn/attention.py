"""Self-attention mixer: fused QKV projection, optional QK-norm, RoPE, GQA, sinks / softcap / window, KV cache.

Capability parity: src/dew/nn/mixers/attention.py:984-1764 (``CausalSelfAttention``), src/dew/nn/rope.py.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, RMSNorm, declare


class SelfAttention(nn.Module):
    def __init__(self, features: int, num_heads: int, num_kv_heads: Optional[int] = None, head_dim: Optional[int] = None,
                 qk_norm: bool = False, bias: bool = False, causal: bool = True, window: Optional[int] = None,
                 softcap: float = 0.0, sinks: bool = False, norm_eps: float = 1e-6, out_zero_init: bool = False,
                 init_std: Optional[float] = None, qkv_bias: bool = False, scale: Optional[float] = None, qk_norm_full: bool = False,
                 out_gate: bool = False, dtype=None, device=None):
        super().__init__()
        self.features, self.num_heads = features, num_heads
        # a softmax scale other than head_dim ** -0.5 is folded into the queries (after the norm and the rotation)
        self.q_gain = None if scale is None else float(scale) * (head_dim or features // num_heads) ** 0.5
        self.num_kv_heads = num_kv_heads or num_heads
        self.head_dim = head_dim or features // num_heads
        self.causal, self.window, self.softcap = causal, window, softcap
        qkv_out = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        self.qkv_proj = Linear(features, qkv_out, bias=bias or qkv_bias, axes=("embed", "heads"), init_std=init_std, dtype=dtype, device=device)
        self.o_proj = Linear(self.num_heads * self.head_dim, features, bias=bias, axes=("heads", "embed"),
                             init_std=init_std, zero_init=out_zero_init, dtype=dtype, device=device)
        # Qwen3-Next: the heads' outputs pass a sigmoid gate computed from the layer's input, before the output projection
        self.gate_proj = Linear(features, self.num_heads * self.head_dim, axes=("embed", "heads"), init_std=init_std, dtype=dtype, device=device) if out_gate else None
        # OLMo-2 normalises q and k over all their heads at once (one weight of heads x head_dim); the usual form is per head
        self.qk_norm_full = qk_norm_full
        qw, kw = (self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim) if qk_norm_full else (self.head_dim, self.head_dim)
        self.q_norm = RMSNorm(qw, norm_eps, dtype=dtype, device=device) if (qk_norm or qk_norm_full) else None
        self.k_norm = RMSNorm(kw, norm_eps, dtype=dtype, device=device) if (qk_norm or qk_norm_full) else None
        self.sinks = declare(nn.Parameter(torch.zeros(num_heads, dtype=dtype, device=device)), ("heads",), "sinks") if sinks else None
        # a layer whose rotary table differs from the model's: (theta, scaling) builds its own; rotary False drops the rotation (NoPE)
        self.rotary, self.own_rope, self._own = True, None, None
        self.head_transform = None     # a module applied to the heads' outputs [B, S, H, D] before the output projection (dew_b200.nn.dex)
        self.track_qk_max = False      # set by dew_b200.optim.qk_clip.watch: record each head's largest attention logit
        self.qk_max: Optional[torch.Tensor] = None

    @torch.no_grad()
    def _record_qk_max(self, q, k):
        """Per query head, the largest visible logit ``scale * q . k`` of this call (exact, computed in key blocks)."""
        B, S, H, D = q.shape
        T, Hkv = k.shape[1], k.shape[2]
        qf = q.float().reshape(B, S, Hkv, H // Hkv, D)
        best = torch.full((H,), float("-inf"), device=q.device)
        qi = torch.arange(S, device=q.device)[:, None] + (T - S)
        for t0 in range(0, T, 1024):
            kb = k[:, t0:t0 + 1024].float()
            s = torch.einsum("bsgrd,btgd->bgrst", qf, kb) * (D ** -0.5)
            if self.causal:
                s = s.masked_fill(~(torch.arange(t0, t0 + kb.shape[1], device=q.device)[None, :] <= qi), float("-inf"))
            best = torch.maximum(best, s.amax((0, 3, 4)).reshape(H))
        self.qk_max = best if self.qk_max is None else torch.maximum(self.qk_max, best)

    def project(self, x, cos=None, sin=None, positions=None):
        B, S, _ = x.shape
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = self.qkv_proj(x).view(B, S, H + 2 * Hkv, D)
        if self.q_norm is not None and self.qk_norm_full:
            q = self.q_norm(qkv[:, :, :H].reshape(B, S, H * D)).view(B, S, H, D)
            k = self.k_norm(qkv[:, :, H:H + Hkv].reshape(B, S, Hkv * D)).view(B, S, Hkv, D)
            qkv = torch.cat([q, k, qkv[:, :, H + Hkv:]], 2)
        elif self.q_norm is not None:
            q = self.q_norm(qkv[:, :, :H])
            k = self.k_norm(qkv[:, :, H:H + Hkv])
            qkv = torch.cat([q, k, qkv[:, :, H + Hkv:]], 2)
        if cos is not None:
            qkv = ops.rope(qkv, cos, sin, positions, rot_heads=H + Hkv)
        q = qkv[:, :, :H]
        return (q if self.q_gain is None else q * self.q_gain), qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]

    def _tables(self, cos, sin):
        if not self.rotary:
            return None, None
        if self.own_rope is None or cos is None:
            return cos, sin
        if self._own is None or self._own[0].device != cos.device or self._own[0].shape[0] != cos.shape[0]:
            theta, scaling = self.own_rope
            self._own = ops.rope_tables(cos.shape[0], self.head_dim, theta, cos.device, scaling)
        return self._own

    def forward(self, x, cos=None, sin=None, positions=None, segment_ids=None, cache=None, layer: int = 0):
        B, S, _ = x.shape
        cos, sin = self._tables(cos, sin)
        if (cache is None and x.is_cuda and cos is not None and self.head_transform is None and self.gate_proj is None and self.q_norm is None and self.window is None and not self.softcap
                and self.sinks is None and segment_ids is None and not self.track_qk_max and self.q_gain is None):
            from ..ops.attn import packed_attention
            H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
            o = packed_attention(self.qkv_proj(x).view(B, S, H + 2 * Hkv, D), cos, sin, positions, H, Hkv, self.causal)
            if o is not None:
                return self.o_proj(o.reshape(B, S, H * D))
        if (cache is not None and S == 1 and self.q_norm is None and self.q_gain is None and positions is not None and cos is not None
                and self.head_transform is None and self.gate_proj is None and hasattr(cache, "decode_packed")):
            # decode step: rotation, cache append and attention straight from the packed projection (no slices, no copies)
            H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
            qkv = self.qkv_proj(x).view(B, H + 2 * Hkv, D)
            if cache.can_decode_packed(qkv, H, self.softcap):
                o = cache.decode_packed(layer, qkv, cos, sin, positions.reshape(-1), H, window=self.window, sinks=self.sinks)
                return self.o_proj(o.reshape(B, 1, H * D))
        q, k, v = self.project(x, cos, sin, positions)
        if self.track_qk_max and cache is None and self.training:
            self._record_qk_max(q, k)
        if cache is None and hasattr(segment_ids, "visible"):
            # rows that share a prefix (dew_b200.data.forked_rows.Forks): a token sees its own document causally and all of its parent
            if self.window is not None or self.softcap or self.sinks is not None or not self.causal:
                raise NotImplementedError("forked rows are built for plain causal attention (no window, soft cap or sinks)")
            from .attention_variants import biased_attention
            o = biased_attention(q, k, v, mask=segment_ids.visible()[:, None])
        elif cache is not None:
            o = cache.attend(layer, q, k, v, positions, causal=self.causal, window=self.window, softcap=self.softcap,
                             sinks=self.sinks)
        else:
            o = ops.attention(q, k, v, causal=self.causal, window=self.window, softcap=self.softcap, sinks=self.sinks,
                              segment_ids=segment_ids)
        if self.head_transform is not None:
            o = self.head_transform(o)
        o = o.reshape(B, S, self.num_heads * self.head_dim)
        if self.gate_proj is not None:
            o = o * torch.sigmoid(self.gate_proj(x).float()).to(o.dtype)
        return self.o_proj(o)
