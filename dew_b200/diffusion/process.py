"""``Process`` = (training schedule, prediction transform, weighting, sampling schedule) and ``Denoiser``.

Parity: src/dew/diffusion/process.py:44-230.  A ``Denoiser`` closes a model over its variables and
conditions and maps ``(x_t, t)`` to ``(x_0 estimate, eps estimate)``; samplers only ever see that.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional, Tuple

import torch

from ..utils import keys as K
from .schedules import NoiseScheduler, expand, times
from .transforms import PredictionTransform, ScheduleWeighting, broadcast_rates


@dataclass(frozen=True)
class Process:
    schedule: NoiseScheduler
    prediction: PredictionTransform
    weighting: Any = ScheduleWeighting()
    sampling: Optional[NoiseScheduler] = None

    def sampler_schedule(self) -> NoiseScheduler:
        return self.sampling if self.sampling is not None else self.schedule

    def weight(self, t) -> torch.Tensor:
        return self.weighting(self.schedule, self.prediction, t)

    def rates(self, t, *, like: torch.Tensor):
        return broadcast_rates(self.schedule, t, like)

    def variances(self, t, *, like: torch.Tensor):
        a, s = self.rates(t, like=like)
        return a * a, s * s

    def times(self, steps: int) -> torch.Tensor:
        """Sampling grid: ``steps + 1`` times from T down to 0 on the sampler schedule."""
        T = self.sampler_schedule().T
        return torch.linspace(T, 0.0, steps + 1, dtype=torch.float64).to(torch.float32)

    def noise(self, key: K.Key, shape) -> torch.Tensor:
        """Prior draw x_T scaled to the sampler schedule's terminal sigma."""
        sched = self.sampler_schedule()
        a, s = sched.rates(torch.tensor(sched.T))
        return K.normal(key, shape) * float(s)

    def denoiser(self, model: Callable, params: Any = None, conditions: Optional[Mapping[str, Any]] = None,
                 *, schedule: Optional[NoiseScheduler] = None, apply: Optional[Callable] = None) -> "Denoiser":
        return Denoiser(self, model, params, dict(conditions or {}), schedule or self.sampler_schedule(), apply)


class Denoiser:
    """``denoiser(x_t, t) -> (x_0, eps)``; ``raw`` exposes the network's untransformed output."""

    def __init__(self, process: Process, model, params, conditions, schedule, apply=None):
        self.process, self.model, self.params = process, model, params
        self.conditions, self.schedule, self.apply = conditions, schedule, apply

    def _call_model(self, x, time, conditions):
        if self.apply is not None:
            return self.apply(self.params, x, time, conditions)
        if self.params is not None and isinstance(self.model, torch.nn.Module):
            from ..utils.trees import variables_for_call
            return torch.func.functional_call(self.model, variables_for_call(self.model, self.params), (x, time, conditions))
        return self.model(x, time, conditions)

    def raw(self, x_t, t, conditions=None):
        t = times(t).to(x_t.device)
        if t.dim() == 0:
            t = t.expand(x_t.shape[0])
        rates = broadcast_rates(self.schedule, t, x_t)
        c_in = self.process.prediction.get_input_scale(rates)
        time = self.schedule.model_time(t)
        return self._call_model(x_t * c_in, time, self.conditions if conditions is None else conditions)

    def convert(self, x_t, t, output):
        t = times(t).to(x_t.device)
        if t.dim() == 0:
            t = t.expand(x_t.shape[0])
        rates = broadcast_rates(self.schedule, t, x_t)
        pred = self.process.prediction.pred_transform(x_t, output, rates, t)
        return self.process.prediction.backward_diffusion(x_t, pred, rates)

    def __call__(self, x_t, t, conditions=None):
        return self.convert(x_t, t, self.raw(x_t, t, conditions))

    def with_conditions(self, conditions) -> "Denoiser":
        return Denoiser(self.process, self.model, self.params, dict(conditions), self.schedule, self.apply)
