"""Noise schedules: ``rates(t) -> (alpha, sigma)``, training-time draws, weights and model time.

Families covered (reference: src/dew/diffusion/schedules/{common,karras,cosine,linear,exp,sqrt,flow}.py):
variance-exploding "generalized" schedules parameterised by sigma (EDM log-normal draw, Karras rho grid),
variance-preserving discrete/continuous cosine and linear-beta schedules, exponential and sqrt schedules,
and the rectified-flow interpolation (with resolution shift).
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

from ..utils import keys as K


def times(t) -> torch.Tensor:
    t = torch.as_tensor(t)
    return t if t.dtype.is_floating_point else t.to(torch.float32)


def expand(coefficient, x: torch.Tensor) -> torch.Tensor:
    """Reshape a per-row coefficient so it broadcasts against ``x``."""
    c = torch.as_tensor(coefficient, device=x.device)
    if c.dim() == 0:
        return c.to(x.dtype if x.dtype.is_floating_point else torch.float32)
    return c.reshape(c.shape[0], *([1] * (x.dim() - 1))).to(x.dtype)


class NoiseScheduler:
    """x_t = alpha(t) x_0 + sigma(t) eps."""
    T: float = 1.0

    def settings(self) -> tuple:
        return tuple(sorted((k, v) for k, v in vars(self).items() if not k.startswith("_")))

    def __eq__(self, other) -> bool:
        return type(self) is type(other) and self.settings() == other.settings()

    def __hash__(self) -> int:
        return hash((type(self).__name__, self.settings()))

    def rates(self, t) -> Tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError

    def sample_t(self, key: K.Key, n: int) -> torch.Tensor:
        return K.uniform(key, (n,)) * self.T

    def weight(self, t) -> torch.Tensor:
        return torch.ones_like(times(t))

    def model_time(self, t) -> torch.Tensor:
        return times(t)

    def prior_scale(self) -> float:
        a, s = self.rates(torch.tensor(self.T))
        return float(s)

    def variances(self, t):
        a, s = self.rates(t)
        return a * a, s * s

    def snr(self, t) -> torch.Tensor:
        a, s = self.rates(t)
        return (a * a) / (s * s).clamp_min(1e-30)


class GeneralizedNoiseScheduler(NoiseScheduler):
    """Variance-exploding: alpha = 1, sigma = sigmas(t); lambda weight and log-sigma/4 model time (EDM)."""

    def __init__(self, sigma_min=0.002, sigma_max=80.0, sigma_data=0.5):
        self.sigma_min, self.sigma_max, self.sigma_data = sigma_min, sigma_max, sigma_data

    def sigma_range(self):
        return self.sigma_min, self.sigma_max

    def sigmas(self, t) -> torch.Tensor:
        raise NotImplementedError

    def t_of_sigma(self, sigma) -> torch.Tensor:
        raise NotImplementedError

    def rates(self, t):
        s = self.sigmas(t)
        return torch.ones_like(s), s

    def weight(self, t):
        s = self.sigmas(t)
        return 1.0 / (self.sigma_data ** 2) + 1.0 / (s * s)

    def model_time(self, t):
        return torch.log(self.sigmas(t)) / 4.0


class KarrasVENoiseScheduler(GeneralizedNoiseScheduler):
    """sigma(t) = (smax^(1/rho) + (1 - t)(smin^(1/rho) - smax^(1/rho)))^rho  (Karras et al. 2022, Eq. 5)."""

    def __init__(self, sigma_min=0.002, sigma_max=80.0, rho=7.0, sigma_data=0.5):
        super().__init__(sigma_min, sigma_max, sigma_data)
        self.rho = float(rho)

    def sigmas(self, t):
        ramp = (1.0 - times(t) / self.T).clamp(0.0, 1.0)
        lo, hi = self.sigma_min ** (1 / self.rho), self.sigma_max ** (1 / self.rho)
        return (hi + ramp * (lo - hi)) ** self.rho

    def t_of_sigma(self, sigma):
        lo, hi = self.sigma_min ** (1 / self.rho), self.sigma_max ** (1 / self.rho)
        ramp = ((times(sigma) ** (1 / self.rho) - hi) / (lo - hi)).clamp(0.0, 1.0)
        return (1.0 - ramp) * self.T


class EDMNoiseScheduler(GeneralizedNoiseScheduler):
    """Training draw: t ~ N(0,1), sigma = exp(P_mean + P_std t)."""

    def __init__(self, sigma_min=0.002, sigma_max=80.0, sigma_data=0.5, P_mean=-0.4, P_std=1.0):
        super().__init__(sigma_min, sigma_max, sigma_data)
        self.P_mean, self.P_std = P_mean, P_std

    def sigmas(self, t):
        return torch.exp(times(t) / self.T * self.P_std + self.P_mean)

    def t_of_sigma(self, sigma):
        return (torch.log(times(sigma)) - self.P_mean) / self.P_std * self.T

    def sample_t(self, key, n):
        return K.normal(key, (n,))


class ExpNoiseScheduler(GeneralizedNoiseScheduler):
    """sigma geometric in t between sigma_min and sigma_max."""

    def sigmas(self, t):
        u = (times(t) / self.T).clamp(0, 1)
        return self.sigma_min * (self.sigma_max / self.sigma_min) ** u

    def t_of_sigma(self, sigma):
        return torch.log(times(sigma) / self.sigma_min) / math.log(self.sigma_max / self.sigma_min) * self.T


class SqrtNoiseScheduler(GeneralizedNoiseScheduler):
    def sigmas(self, t):
        u = (times(t) / self.T).clamp(0, 1)
        return self.sigma_min + (self.sigma_max - self.sigma_min) * torch.sqrt(u)

    def t_of_sigma(self, sigma):
        return ((times(sigma) - self.sigma_min) / (self.sigma_max - self.sigma_min)) ** 2 * self.T


class CosineContinuousNoiseScheduler(NoiseScheduler):
    """alpha = cos(pi t / 2), sigma = sin(pi t / 2) on t in [0, 1]."""

    def __init__(self, eps: float = 1e-4):
        self.eps = eps

    def rates(self, t):
        u = (times(t) / self.T).clamp(self.eps, 1 - self.eps)
        return torch.cos(u * math.pi / 2), torch.sin(u * math.pi / 2)

    def weight(self, t):
        return torch.ones_like(times(t))


class CosineNoiseScheduler(NoiseScheduler):
    """Nichol & Dhariwal discrete cosine schedule with ``timesteps`` steps (t integer-valued in [0, T])."""

    def __init__(self, timesteps: int = 1000, s: float = 0.008):
        self.timesteps, self.s = timesteps, s
        self.T = float(timesteps)

    def _alpha_bar(self, t):
        u = (times(t) / self.T).clamp(0, 1)
        f = torch.cos((u + self.s) / (1 + self.s) * math.pi / 2) ** 2
        f0 = math.cos(self.s / (1 + self.s) * math.pi / 2) ** 2
        return (f / f0).clamp(1e-8, 1.0)

    def rates(self, t):
        ab = self._alpha_bar(t)
        return torch.sqrt(ab), torch.sqrt(1 - ab)

    def sample_t(self, key, n):
        return K.randint(key, (n,), 1, self.timesteps + 1).to(torch.float32)


class LinearNoiseScheduler(NoiseScheduler):
    """DDPM linear-beta schedule in its continuous (VP-SDE) form."""

    def __init__(self, timesteps: int = 1000, beta_start: float = 1e-4, beta_end: float = 0.02):
        self.timesteps, self.beta_start, self.beta_end = timesteps, beta_start, beta_end
        self.T = float(timesteps)

    def rates(self, t):
        u = (times(t) / self.T).clamp(0, 1)
        b0, b1 = self.beta_start * self.timesteps, self.beta_end * self.timesteps
        log_ab = -(b0 * u + 0.5 * (b1 - b0) * u * u)
        ab = torch.exp(log_ab)
        return torch.sqrt(ab), torch.sqrt((1 - ab).clamp_min(1e-12))

    def sample_t(self, key, n):
        return K.randint(key, (n,), 1, self.timesteps + 1).to(torch.float32)


class FlowNoiseScheduler(NoiseScheduler):
    """Rectified flow: x_t = (1 - t) x_0 + t eps; optional resolution shift and logit-normal draw."""

    def __init__(self, shift: float = 1.0, logit_normal: bool = False, mean: float = 0.0, std: float = 1.0):
        self.shift, self.logit_normal, self.mean, self.std = shift, logit_normal, mean, std

    def _shifted(self, t):
        t = times(t)
        return self.shift * t / (1 + (self.shift - 1) * t)

    def rates(self, t):
        u = self._shifted(t).clamp(0, 1)
        return 1 - u, u

    def sample_t(self, key, n):
        if self.logit_normal:
            return torch.sigmoid(K.normal(key, (n,)) * self.std + self.mean)
        return K.uniform(key, (n,))
