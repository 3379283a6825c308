"""Activation statistics a run watches: forward hooks on chosen modules record, per call, the output's RMS, mean, largest magnitude,
share of exact zeros, excess kurtosis over channels (heavy tails announce outlier channels long before a loss spike) and the channel
that carries the largest RMS.  ``ActivationWatch`` is a context manager; ``collect()`` returns plain floats keyed by module path, ready
for a metrics log, and clears what it held.  The statistics are computed in fp32 on the device and read back only in ``collect``, so
watching costs a few reductions per watched module and no synchronisation in the step.

Reference: src/dew/nn/inspection.py.
"""
from __future__ import annotations

import fnmatch
from typing import Dict, Iterable, List, Optional, Sequence

import torch
import torch.nn as nn


def activation_statistics(y: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Statistics of one activation ``[..., channels]`` as 0-d fp32 tensors on its device."""
    f = y.detach().float()
    flat = f.reshape(-1, f.shape[-1]) if f.dim() > 1 else f.reshape(-1, 1)
    mean, var = flat.mean(), flat.var(unbiased=False)
    centred = flat - mean
    kurt = (centred ** 4).mean() / var.clamp_min(1e-30) ** 2 - 3.0
    per_channel = flat.pow(2).mean(0).sqrt()
    top = per_channel.argmax()
    return {"rms": flat.pow(2).mean().sqrt(), "mean": mean, "max_abs": flat.abs().max(), "zeros": (flat == 0).float().mean(),
            "kurtosis": kurt, "top_channel": top.float(), "top_channel_rms": per_channel[top]}


class ActivationWatch:
    """``with ActivationWatch(model, ["layers.*.mlp", "final_norm"]) as watch: ...; watch.collect()``.

    ``patterns`` are shell-style patterns over ``named_modules`` paths.  A module called several times between two ``collect`` calls
    (gradient accumulation, a looped block) reports the mean of its calls, and ``calls`` says how many there were."""

    def __init__(self, model: nn.Module, patterns: Sequence[str] = ("*",), leaves_only: bool = True):
        self.model, self.patterns, self.leaves_only = model, list(patterns), leaves_only
        self._handles: List[torch.utils.hooks.RemovableHandle] = []
        self._held: Dict[str, List[Dict[str, torch.Tensor]]] = {}

    def watched(self) -> List[str]:
        names = []
        for name, module in self.model.named_modules():
            if not name or (self.leaves_only and any(True for _ in module.children()) and not any(fnmatch.fnmatchcase(name, p) and p != "*" for p in self.patterns)):
                continue
            if any(fnmatch.fnmatchcase(name, p) for p in self.patterns):
                names.append(name)
        return names

    def __enter__(self) -> "ActivationWatch":
        modules = dict(self.model.named_modules())
        for name in self.watched():
            def hook(_module, _inputs, output, name=name):
                out = output[0] if isinstance(output, (tuple, list)) else output
                if torch.is_tensor(out) and out.is_floating_point() and out.numel():
                    self._held.setdefault(name, []).append(activation_statistics(out))
            self._handles.append(modules[name].register_forward_hook(hook))
        return self

    def __exit__(self, *exc) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    def collect(self) -> Dict[str, float]:
        out: Dict[str, float] = {}
        for name, calls in self._held.items():
            for key in calls[0]:
                vals = torch.stack([c[key] for c in calls])
                out[f"{name}/{key}"] = float(vals[-1] if key == "top_channel" else vals.mean())
            out[f"{name}/calls"] = float(len(calls))
        self._held = {}
        return out


def outliers(stats: Dict[str, float], kurtosis: float = 20.0, ratio: float = 8.0) -> List[str]:
    """Module paths whose last collection shows heavy tails: excess kurtosis above ``kurtosis`` or one channel's RMS above ``ratio`` times the tensor's."""
    names = sorted({k.rsplit("/", 1)[0] for k in stats})
    return [n for n in names if stats.get(f"{n}/kurtosis", 0.0) > kurtosis or stats.get(f"{n}/top_channel_rms", 0.0) > ratio * max(stats.get(f"{n}/rms", 0.0), 1e-30)]
