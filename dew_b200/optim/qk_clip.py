"""QK-clip (MuonClip, Kimi K2): after an optimizer step, shrink the query and key projections of every attention head whose
largest logit of the step exceeded ``tau``, so the logits cannot run away under Muon's large updates.

``watch(model)`` asks the attention layers to record each head's largest logit; ``qk_clip(model, tau)`` reads and clears
those records and rescales, per key / value group ``g`` (grouped-query attention shares a key head among its query heads):
``gamma_g = min(1, tau / max_{h in g} S_max_h)``, the group's key rows and its query heads' rows each times ``sqrt(gamma_g)``,
so every logit of the group shrinks by ``gamma_g``.  Layers with q/k normalisation are left alone: their logits are bounded
by the norm's scale.  Returns the per-layer maxima for logging.

Reference: src/dew/optim.py (``scale_by_qk_clip`` :750, ``_clip_scale`` :515, ``_qk_normed`` :566, ``_muonclip_groups`` :937).
"""
from __future__ import annotations

from typing import Dict

import torch


def _layers(model: torch.nn.Module):
    from ..nn.attention import SelfAttention
    for name, m in model.named_modules():
        if isinstance(m, SelfAttention) and m.q_norm is None:
            yield name, m


def watch(model: torch.nn.Module, on: bool = True) -> int:
    """Turn the recording on (or off); returns how many layers are watched."""
    n = 0
    for _, m in _layers(model):
        m.track_qk_max, m.qk_max = on, None
        n += 1
    return n


@torch.no_grad()
def qk_clip(model: torch.nn.Module, tau: float = 100.0) -> Dict[str, torch.Tensor]:
    if not tau > 0:
        raise ValueError(f"tau bounds the attention logits, so it is positive, got {tau}")
    seen = {}
    for name, m in _layers(model):
        if m.qk_max is None:
            continue
        H, Hkv, D = m.num_heads, m.num_kv_heads, m.head_dim
        s_max = m.qk_max.float()
        seen[name] = s_max.clone()
        group_max = s_max.reshape(Hkv, H // Hkv).amax(1)
        gamma = torch.clamp(tau / group_max.clamp_min(1e-20), max=1.0)             # [Hkv]
        if bool((gamma < 1).any()):
            root = gamma.sqrt()
            w = m.qkv_proj.weight                                                    # [(H + 2 Hkv) D, features]
            rows = w.view(H + 2 * Hkv, D, -1)
            rows[:H].mul_(root.repeat_interleave(H // Hkv)[:, None, None].to(w.dtype))
            rows[H:H + Hkv].mul_(root[:, None, None].to(w.dtype))
            b = getattr(m.qkv_proj, "bias", None)
            if b is not None:
                bv = b.view(H + 2 * Hkv, D)
                bv[:H].mul_(root.repeat_interleave(H // Hkv)[:, None].to(b.dtype))
                bv[H:H + Hkv].mul_(root[:, None].to(b.dtype))
        m.qk_max = None
    return seen
