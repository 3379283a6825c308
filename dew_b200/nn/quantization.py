"""Weight quantisation for inference: int8 / fp8-e4m3 per-output-channel, and NVFP4-style 4-bit blocks of 16 with
e4m3 block scales; ``Quantization`` config, ``quantize_variables`` (post-training), ``fake_quant`` (QAT straight-through).

Reference: src/dew/quantization.py (PTQ / QAT; int8, fp8), src/dew/nn/kernels/templates/gemm/formats.py (``NvFp4`` :29,
``MxFp8`` :186), src/dew/nn/fake_quant.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

import torch

from ..utils.trees import flatten, unflatten

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


@dataclass(frozen=True)
class Quantization:
    kind: str = "int8"                 # int8 | float8_e4m3fn | nvfp4
    min_size: int = 4096               # leaves smaller than this stay as they are
    skip: Tuple[str, ...] = ("embed", "norm", "scale", "bias", "router")


def quantize_weight(w: torch.Tensor, kind: str) -> Dict[str, torch.Tensor]:
    """``w [out, in]`` -> stored tensors; ``dequantize_weight`` inverts (up to rounding)."""
    wf = w.float()
    if kind == "int8":
        scale = wf.abs().amax(1, keepdim=True).clamp_min(1e-12) / 127.0
        return {"q": (wf / scale).round().clamp(-127, 127).to(torch.int8), "scale": scale.squeeze(1)}
    if kind == "float8_e4m3fn":
        scale = wf.abs().amax(1, keepdim=True).clamp_min(1e-12) / 448.0
        return {"q": (wf / scale).to(torch.float8_e4m3fn), "scale": scale.squeeze(1)}
    if kind == "nvfp4":
        out, inn = wf.shape
        pad = (-inn) % 16
        if pad:
            wf = torch.nn.functional.pad(wf, (0, pad))
        blocks = wf.reshape(out, -1, 16)
        tensor_scale = wf.abs().amax().clamp_min(1e-12) / (6.0 * 448.0)
        bscale = (blocks.abs().amax(-1) / 6.0 / tensor_scale).to(torch.float8_e4m3fn)       # e4m3 block scales
        denom = (bscale.float() * tensor_scale).clamp_min(1e-12)[..., None]
        mag = (blocks.abs() / denom)
        idx = (mag[..., None] - E2M1_VALUES.to(w.device)).abs().argmin(-1).to(torch.uint8)   # nearest e2m1 magnitude
        code = idx | ((blocks < 0).to(torch.uint8) << 3)
        packed = (code[..., 0::2] | (code[..., 1::2] << 4)).reshape(out, -1)
        return {"q": packed, "block_scale": bscale, "tensor_scale": tensor_scale.reshape(()), "in_features": torch.tensor(inn)}
    raise ValueError(f"unknown quantisation kind {kind!r}")


def dequantize_weight(stored: Mapping[str, torch.Tensor], kind: str, dtype=torch.float32) -> torch.Tensor:
    if kind in ("int8", "float8_e4m3fn"):
        return (stored["q"].float() * stored["scale"][:, None]).to(dtype)
    if kind == "nvfp4":
        packed = stored["q"]
        out = packed.shape[0]
        lo, hi = packed & 0xF, packed >> 4
        code = torch.stack([lo, hi], -1).reshape(out, -1, 16)
        mag = E2M1_VALUES.to(packed.device)[(code & 7).long()]
        val = torch.where((code & 8) > 0, -mag, mag)
        w = val * (stored["block_scale"].float() * stored["tensor_scale"])[..., None]
        return w.reshape(out, -1)[:, : int(stored["in_features"])].to(dtype)
    raise ValueError(kind)


def quantize_variables(variables: Mapping[str, Any], q: Quantization) -> Dict[str, Any]:
    """Round-trip every eligible 2-D weight through its quantised form (weights stay in their dtype, carrying the
    quantisation error), so any model runs unchanged on the result."""
    flat = flatten(variables)
    out = {}
    for path, t in flat.items():
        if isinstance(t, torch.Tensor) and t.dim() == 2 and t.numel() >= q.min_size and not any(s in path for s in q.skip):
            out[path] = dequantize_weight(quantize_weight(t, q.kind), q.kind, t.dtype)
        else:
            out[path] = t
    return unflatten(out)


class _FakeQuant(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, kind):
        return dequantize_weight(quantize_weight(w, kind), kind, w.dtype)

    @staticmethod
    def backward(ctx, g):
        return g, None           # straight-through estimator


def fake_quant(w: torch.Tensor, kind: str = "int8") -> torch.Tensor:
    return _FakeQuant.apply(w, kind)
