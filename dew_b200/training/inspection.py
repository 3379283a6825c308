"""Live inspection of a run's parameters and updates: every ``every`` steps the inspector keeps the parameters' norms per group (a
layer, the embedding, the head ...), and one step later the size of the update each group took, as an RMS and as a ratio to the
parameters' own RMS - the number that says whether a layer is learning at the rate the others are (ratios near 1e-3 are healthy for
Adam at usual rates; a group orders of magnitude above is about to diverge, one orders below is frozen in effect).  Passed to
``Trainer.fit`` twice: ``observe=inspector`` (called every step, cheap unless it is a step to look at) and
``summaries=inspector.summaries`` (the latest numbers, logged beside the loss).

Reference: src/dew/training/inspection.py.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Mapping, Optional

import torch

from ..utils.trees import flatten


def group_of(path: str, depth: int = 2) -> str:
    """``layers.3.mixer.qkv_proj.weight`` -> ``layers.3``; ``layers_3/mixer/qkv_proj/weight`` (a train state's paths) -> ``layers_3``;
    ``embed.weight`` -> ``embed``."""
    parts = path.replace("/", ".").split(".")
    if parts and parts[0] == "params":
        parts = parts[1:]
    keep = parts[:depth] if len(parts) > depth and parts[min(1, len(parts) - 1)].isdigit() else parts[:1]
    return ".".join(keep)


def _sums(flat: Mapping[str, torch.Tensor], depth: int) -> Dict[str, List[float]]:
    out: Dict[str, List[float]] = {}
    for path, p in flat.items():
        if not torch.is_tensor(p) or not p.is_floating_point():
            continue
        g = out.setdefault(group_of(path, depth), [0.0, 0.0])
        g[0] += float(p.detach().float().pow(2).sum())
        g[1] += p.numel()
    return out


class RunInspector:
    def __init__(self, every: int = 100, depth: int = 2, params_of: Optional[Callable[[Any], Mapping[str, Any]]] = None):
        self.every, self.depth = max(1, every), depth
        self.params_of = params_of or (lambda state: state.variables.get("params", state.variables))
        self._before: Optional[Dict[str, torch.Tensor]] = None
        self._before_step = -1
        self.latest: Dict[str, float] = {}
        self.rows: List[Dict[str, float]] = []

    def __call__(self, state, metrics=None) -> None:
        step = int(state.step)
        if self._before is not None and step == self._before_step + 1:
            self._compare(flatten(self.params_of(state)), step)
            self._before = None
        if step % self.every == 0:
            self._before = {k: v.detach().clone() for k, v in flatten(self.params_of(state)).items() if torch.is_tensor(v) and v.is_floating_point()}
            self._before_step = step

    def _compare(self, now: Mapping[str, torch.Tensor], step: int) -> None:
        before = self._before
        params = _sums(now, self.depth)
        delta = _sums({k: now[k].detach().float() - v.float() for k, v in before.items() if k in now}, self.depth)
        row: Dict[str, float] = {"step": float(step)}
        worst, worst_ratio = "", 0.0
        for g, (sq, n) in params.items():
            rms = (sq / max(1, n)) ** 0.5
            upd = (delta.get(g, [0.0, 1])[0] / max(1, n)) ** 0.5
            ratio = upd / max(rms, 1e-30)
            row[f"inspect/{g}/param_rms"], row[f"inspect/{g}/update_rms"], row[f"inspect/{g}/update_ratio"] = rms, upd, ratio
            if ratio > worst_ratio:
                worst, worst_ratio = g, ratio
        row["inspect/max_update_ratio"] = worst_ratio
        self.latest, self.worst_group = row, worst
        self.rows.append(row)

    def summaries(self, state=None) -> Dict[str, float]:
        return {k: v for k, v in self.latest.items() if k != "step"}
