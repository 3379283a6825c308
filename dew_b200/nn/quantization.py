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


# ---------------------------------------------------------------------------------------------------------------
# Quantised modules (weights stay quantised in memory), QAT wrappers and activation calibration
import torch.nn as nn  # noqa: E402


class QuantizedLinear(nn.Module):
    """A ``Linear`` whose weight lives in memory in its quantised form.  fp8 weights on a GPU multiply through the
    row-scaled e4m3 tensor-core GEMM (activations quantised per row on the way in); every other case de-quantises the
    weight for the call.  ``from_linear`` quantises an existing layer."""

    def __init__(self, in_features: int, out_features: int, kind: str, stored: Mapping[str, torch.Tensor], bias=None, dtype=torch.bfloat16):
        super().__init__()
        self.in_features, self.out_features, self.kind, self.dtype = in_features, out_features, kind, dtype
        for k, v in stored.items():
            self.register_buffer(f"q_{k}", v)
        self.bias = bias

    @classmethod
    def from_linear(cls, lin, kind: str) -> "QuantizedLinear":
        return cls(lin.in_features, lin.out_features, kind, quantize_weight(lin.weight.detach(), kind), lin.bias, lin.weight.dtype)

    def stored(self) -> Dict[str, torch.Tensor]:
        return {k[2:]: v for k, v in self._buffers.items() if k.startswith("q_")}

    @property
    def weight(self) -> torch.Tensor:
        return dequantize_weight(self.stored(), self.kind, self.dtype)

    def bytes(self) -> int:
        return sum(v.numel() * v.element_size() for v in self.stored().values())

    def forward(self, x):
        from .. import ops
        if self.kind == "float8_e4m3fn" and x.is_cuda and x.dtype == torch.bfloat16 and self.in_features % 16 == 0:
            from ..ops.fp8 import gemm_fp8, quantize_rows
            x2 = x.reshape(-1, self.in_features)
            xq, xs = quantize_rows(x2)
            y = gemm_fp8(xq, xs, self.q_q, self.q_scale).reshape(*x.shape[:-1], self.out_features)
            return y if self.bias is None else y + self.bias
        return ops.linear(x, self.weight.to(x.dtype), self.bias)


def quantize_model(model: nn.Module, q: Quantization) -> Dict[str, int]:
    """Replace every eligible ``Linear`` of ``model`` in place by a ``QuantizedLinear``; returns bytes before / after."""
    from .layers import Linear
    before = after = 0
    for path, module in list(model.named_modules()):
        for name, child in list(module.named_children()):
            full = f"{path}.{name}" if path else name
            if isinstance(child, Linear) and child.weight.numel() >= q.min_size and not any(s in full for s in q.skip):
                ql = QuantizedLinear.from_linear(child, q.kind)
                before += child.weight.numel() * child.weight.element_size()
                after += ql.bytes()
                setattr(module, name, ql)
    return {"bytes_before": before, "bytes_after": after}


class QATLinear(nn.Module):
    """Quantisation-aware training: the forward sees the weight after a quantise / de-quantise round trip, the backward passes
    straight through to the full-precision weight, which keeps training."""

    def __init__(self, base, kind: str = "int8"):
        super().__init__()
        self.base, self.kind = base, kind

    @property
    def weight(self):
        return self.base.weight

    def forward(self, x):
        from .. import ops
        return ops.linear(x, fake_quant(self.base.weight, self.kind), self.base.bias)


def prepare_qat(model: nn.Module, q: Quantization) -> int:
    from .layers import Linear
    n = 0
    for path, module in list(model.named_modules()):
        for name, child in list(module.named_children()):
            full = f"{path}.{name}" if path else name
            if isinstance(child, Linear) and child.weight.numel() >= q.min_size and not any(s in full for s in q.skip):
                setattr(module, name, QATLinear(child, q.kind))
                n += 1
    return n


def convert_qat(model: nn.Module) -> int:
    """After QAT: every ``QATLinear`` becomes a ``QuantizedLinear`` of the weights it trained."""
    n = 0
    for module in list(model.modules()):
        for name, child in list(module.named_children()):
            if isinstance(child, QATLinear):
                setattr(module, name, QuantizedLinear.from_linear(child.base, child.kind))
                n += 1
    return n


class Calibrator:
    """Static activation ranges: run representative batches with ``observe(model)`` active and read ``scales()`` - the absolute
    maximum each ``Linear`` saw at its input over the calibration set, divided by the format's largest value."""

    def __init__(self, kind: str = "float8_e4m3fn"):
        self.limit = {"int8": 127.0, "float8_e4m3fn": 448.0, "nvfp4": 6.0}[kind]
        self.amax: Dict[str, float] = {}
        self._hooks = []

    def observe(self, model: nn.Module):
        from .layers import Linear
        for name, m in model.named_modules():
            if isinstance(m, (Linear, QuantizedLinear)):
                def hook(mod, args, name=name):
                    self.amax[name] = max(self.amax.get(name, 0.0), float(args[0].detach().abs().amax()))
                self._hooks.append(m.register_forward_pre_hook(hook))
        return self

    def close(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def scales(self) -> Dict[str, float]:
        return {k: (v / self.limit if v > 0 else 1.0) for k, v in self.amax.items()}
