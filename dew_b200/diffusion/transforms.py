"""Prediction transforms (what the network's output means) and loss weightings.

Parity: src/dew/diffusion/transforms.py (Epsilon/Direct/V/FlowMatch/Karras transforms,
ConsistencyBoundary, ScheduleWeighting, MinSNR, VelocityLoss, ``broadcast_rates``).
"""
from __future__ import annotations

from typing import Tuple

import torch

from .schedules import NoiseScheduler, expand, times


def broadcast_rates(schedule: NoiseScheduler, t, x: torch.Tensor):
    a, s = schedule.rates(t)
    return expand(a.to(x.device), x), expand(s.to(x.device), x)


def from_clean(x_t, x_0, rates):
    """(x_0, eps) given the clean estimate."""
    a, s = rates
    return x_0, (x_t - a * x_0) / s.clamp_min(1e-20)


class PredictionTransform:
    def __init__(self, *, normalize_input: bool = False):
        self.normalize_input = normalize_input

    def divides_by_signal(self) -> bool:
        return False

    def pred_transform(self, x_t, prediction, rates, t):
        """Map the raw network output into the space the target lives in."""
        return prediction

    def forward_diffusion(self, x_0, epsilon, rates) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        a, s = rates
        x_t = a * x_0 + s * epsilon
        return x_t, self.get_input_scale(rates), self.get_target(x_0, epsilon, rates)

    def backward_diffusion(self, x_t, prediction, rates):
        """(x_0 estimate, eps estimate) from a transformed prediction."""
        raise NotImplementedError

    def get_target(self, x_0, epsilon, rates):
        return x_0

    def get_input_scale(self, rates):
        if self.normalize_input:
            a, s = rates
            return 1.0 / torch.sqrt(a * a + s * s)
        return torch.ones_like(rates[0])

    def target_error_scale(self, snr):
        """d(target error)/d(x_0 error) squared, used by MinSNR-style weightings."""
        return torch.ones_like(snr)


class EpsilonPredictionTransform(PredictionTransform):
    def divides_by_signal(self):
        return True

    def backward_diffusion(self, x_t, prediction, rates):
        a, s = rates
        return (x_t - s * prediction) / a.clamp_min(1e-20), prediction

    def get_target(self, x_0, epsilon, rates):
        return epsilon

    def target_error_scale(self, snr):
        return snr


class DirectPredictionTransform(PredictionTransform):
    def backward_diffusion(self, x_t, prediction, rates):
        return from_clean(x_t, prediction, rates)


class VPredictionTransform(PredictionTransform):
    def backward_diffusion(self, x_t, prediction, rates):
        a, s = rates
        norm = a * a + s * s
        x_0 = (a * x_t - s * prediction) / norm
        eps = (s * x_t + a * prediction) / norm
        return x_0, eps

    def get_target(self, x_0, epsilon, rates):
        a, s = rates
        return a * epsilon - s * x_0

    def target_error_scale(self, snr):
        return snr + 1


class FlowMatchPredictionTransform(PredictionTransform):
    """Velocity target eps - x_0 on the rectified-flow interpolation."""

    def backward_diffusion(self, x_t, prediction, rates):
        a, s = rates
        x_0 = x_t - s * prediction
        return x_0, x_t + a * prediction

    def get_target(self, x_0, epsilon, rates):
        return epsilon - x_0

    def target_error_scale(self, snr):
        return torch.ones_like(snr)


class KarrasPredictionTransform(PredictionTransform):
    """EDM preconditioning: D = c_skip x + c_out F(c_in x, log(sigma)/4)."""

    def __init__(self, sigma_data: float = 0.5, *, velocity: bool = False):
        super().__init__()
        self.sigma_data, self.velocity = sigma_data, velocity

    def backward_diffusion(self, x_t, prediction, rates):
        return from_clean(x_t, prediction, rates)

    def pred_transform(self, x_t, prediction, rates, t):
        _, s = rates
        sd2 = self.sigma_data ** 2
        c_skip = sd2 / (sd2 + s * s)
        c_out = s * self.sigma_data / torch.sqrt(sd2 + s * s)
        return c_skip * x_t + c_out * prediction

    def get_input_scale(self, rates):
        _, s = rates
        return 1.0 / torch.sqrt(self.sigma_data ** 2 + s * s)


class ConsistencyBoundary(PredictionTransform):
    """Wraps a transform so the model is the identity at t -> 0 (consistency models)."""

    def __init__(self, inner: PredictionTransform, timestep_scaling: float = 10.0, sigma_data: float = 0.5):
        super().__init__()
        self.inner, self.timestep_scaling, self.sigma_data = inner, timestep_scaling, sigma_data

    def pred_transform(self, x_t, prediction, rates, t):
        inner = self.inner.pred_transform(x_t, prediction, rates, t)
        x_0, _ = self.inner.backward_diffusion(x_t, inner, rates)
        st = expand(times(t).to(x_t.device), x_t) * self.timestep_scaling
        sd2 = self.sigma_data ** 2
        c_skip = sd2 / (st * st + sd2)
        c_out = st / torch.sqrt(st * st + sd2)
        return c_skip * x_t + c_out * x_0

    def divides_by_signal(self):
        return self.inner.divides_by_signal()

    def backward_diffusion(self, x_t, prediction, rates):
        return from_clean(x_t, prediction, rates)

    def get_input_scale(self, rates):
        return self.inner.get_input_scale(rates)


class ScheduleWeighting:
    """The schedule's own weight (EDM's lambda for Karras schedules, 1 otherwise)."""

    def __call__(self, schedule, prediction, t):
        return schedule.weight(t)


class MinSNR:
    """min(snr, gamma) weighting in x_0-error units, converted to the prediction's target units."""

    def __init__(self, gamma: float = 5.0):
        self.gamma = gamma

    def __call__(self, schedule, prediction, t):
        snr = schedule.snr(t)
        return torch.minimum(snr, torch.full_like(snr, self.gamma)) / prediction.target_error_scale(snr).clamp_min(1e-20)


class VelocityLoss:
    """Weights a clean-sample prediction's error as a velocity error (1/sigma^2 on flow paths)."""

    def __init__(self, floor: float = 0.05):
        self.floor = floor

    def __call__(self, schedule, prediction, t):
        _, s = schedule.rates(t)
        return 1.0 / (s.clamp_min(self.floor) ** 2)
