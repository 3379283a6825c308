"""``TrainState``: everything a run carries from step to step.

Fields mirror src/dew/state.py:191-280 (step, microstep, updates, variables, opt_state, ema, key, scale,
accumulation, consumed, deferred, inner, compute); ``CHECKPOINTED`` and ``MODEL_STATE`` (:298, :320) say what a
checkpoint stores and which subset serves evaluation / export.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields, replace
from typing import Any, Dict, Mapping, Optional

import torch

CHECKPOINTED = ("step", "microstep", "updates", "variables", "opt_state", "ema", "key", "scale", "accumulation",
                "consumed", "inner")
MODEL_STATE = ("step", "microstep", "updates", "variables", "ema")


@dataclass
class TrainState:
    step: int = 0                     # optimizer steps taken
    microstep: int = 0                # microbatches seen (>= step under accumulation)
    updates: int = 0                  # accepted updates (skip_nonfinite may reject steps)
    variables: Dict[str, Any] = field(default_factory=dict)    # {'params': tree, ...}: the fp32 masters
    opt_state: Dict[str, Any] = field(default_factory=dict)
    ema: Optional[Dict[str, Any]] = None
    key: int = 0
    scale: Optional[Dict[str, Any]] = None       # dynamic loss scale {'scale', 'good_steps'}
    accumulation: Optional[Dict[str, Any]] = None
    consumed: Dict[str, int] = field(default_factory=lambda: {"examples": 0, "tokens": 0})
    deferred: Optional[Any] = None
    inner: Optional[Any] = None                  # DiLoCo inner replicas
    compute: Optional[Dict[str, Any]] = None     # bf16 compute copies (not checkpointed)

    @property
    def averaged(self) -> Dict[str, Any]:
        """EMA variables if an average is kept, else the live ones."""
        return self.ema if self.ema is not None else self.variables

    @property
    def params(self):
        return self.variables.get("params", {})

    def replace(self, **kw) -> "TrainState":
        return replace(self, **kw)

    def checkpointed(self, model_only: bool = False) -> Dict[str, Any]:
        names = MODEL_STATE if model_only else CHECKPOINTED
        return {n: getattr(self, n) for n in names if getattr(self, n) is not None}
