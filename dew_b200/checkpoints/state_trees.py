"""Tree <-> stored-leaf conversions: Flax-style leaf naming and the EMA XOR byte-plane encoding.

* Naming: a PyTorch ``Linear.weight [out, in]`` is stored as ``kernel [in, out]``, a norm's ``weight`` as ``scale``,
  an embedding table as ``embedding`` - the leaf names and orientations of the reference's PyTree, so tree paths
  read ``variables/params/<module path>/kernel`` (Appendix: src/dew/checkpoints/_payloads.py, _state_trees.py).
* EMA planes: an EMA leaf with its weight's dtype and shape is stored as ``bits(ema) XOR bits(weight)`` split into
  byte planes (leading uint8 axis, least-significant byte first); agreeing high bits become zero bytes that
  compress well, and decoding is bit-exact (src/dew/checkpoints/_state_trees.py:117-135).
"""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch

from ..utils.trees import flatten, unflatten

_INT_OF = {4: torch.int32, 2: torch.int16, 8: torch.int64, 1: torch.uint8}
_RENAME = {"kernel": "kernel", "scale": "scale", "embedding": "embedding", "bias": "bias"}


def leaf_kinds(module: torch.nn.Module) -> Dict[str, str]:
    """tree path -> declared kind (``kernel`` / ``scale`` / ``embedding`` / ``bias`` / other)."""
    from ..utils.trees import module_path_to_tree_path
    return {module_path_to_tree_path(n): getattr(p, "dew_kind", "") for n, p in module.named_parameters()}


def to_stored(params: Mapping[str, Any], kinds: Optional[Mapping[str, str]]) -> Dict[str, torch.Tensor]:
    """Flat ``stored path -> tensor`` with Flax leaf names and orientations."""
    out = {}
    for path, t in flatten(params).items():
        kind = (kinds or {}).get(path, "")
        head, _, leaf = path.rpartition("/")
        if kind == "kernel" and t.dim() == 2:
            out[f"{head}/kernel" if head else "kernel"] = t.detach().t()
        elif kind in ("scale", "embedding") and leaf == "weight":
            out[f"{head}/{kind}" if head else kind] = t.detach()
        else:
            out[path] = t.detach() if isinstance(t, torch.Tensor) else t
    return out


def from_stored(stored: Mapping[str, torch.Tensor], kinds: Optional[Mapping[str, str]], template_paths) -> Dict[str, Any]:
    """Inverse of :func:`to_stored` for the parameter paths in ``template_paths``."""
    out = {}
    for path in template_paths:
        kind = (kinds or {}).get(path, "")
        head, _, leaf = path.rpartition("/")
        if kind == "kernel":
            key = f"{head}/kernel" if head else "kernel"
            if key in stored:
                t = stored[key]
                out[path] = t.t().contiguous() if t.dim() == 2 else t
                continue
        if kind in ("scale", "embedding") and leaf == "weight":
            key = f"{head}/{kind}" if head else kind
            if key in stored:
                out[path] = stored[key]
                continue
        if path in stored:
            out[path] = stored[path]
        else:
            raise KeyError(f"checkpoint has no leaf for {path!r}")
    return out


def delta_planes(ema: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``[bytes, *shape]`` uint8 planes of ``bits(ema) ^ bits(weight)``, least-significant byte first."""
    assert ema.dtype == weight.dtype and ema.shape == weight.shape
    it = _INT_OF[ema.element_size()]
    x = ema.detach().cpu().contiguous().view(it) ^ weight.detach().cpu().contiguous().view(it)
    return x.reshape(-1).view(torch.uint8).reshape(*ema.shape, ema.element_size()).movedim(-1, 0).contiguous()


def from_delta_planes(planes: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    it = _INT_OF[weight.element_size()]
    x = planes.movedim(0, -1).contiguous().reshape(-1).view(it).reshape(weight.shape)
    return (x ^ weight.detach().cpu().contiguous().view(it)).view(weight.dtype)


def encode_ema(ema: Mapping[str, torch.Tensor], weights: Mapping[str, torch.Tensor]) -> Tuple[Dict[str, torch.Tensor], List[str]]:
    out, encoded = {}, []
    for path, e in ema.items():
        w = weights.get(path)
        if isinstance(e, torch.Tensor) and w is not None and e.dtype == w.dtype and e.shape == w.shape \
                and e.dtype.is_floating_point and e.numel() > 0:
            out[path] = delta_planes(e, w)
            encoded.append(path)
        else:
            out[path] = e
    return out, encoded


def decode_ema(stored: Mapping[str, torch.Tensor], weights: Mapping[str, torch.Tensor], encoded) -> Dict[str, torch.Tensor]:
    enc = set(encoded)
    return {p: (from_delta_planes(t, weights[p]) if p in enc else t) for p, t in stored.items()}
