"""Process presets: ``EDM``, ``Karras``, ``Cosine``, ``CosineContinuous``, ``Linear``, ``Exp``, ``Sqrt``,
``Flow``, ``ResolutionShift``, ``JiT``, ``MeanFlow``, ``Shortcut``.  Calling a preset builds its ``Process``.

Parity: src/dew/diffusion/presets.py:94-396 (EDM regimes pixel -1.2/1.2 and latent -0.4/1.0; Karras rho grid).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .process import Process
from .schedules import (CosineContinuousNoiseScheduler, CosineNoiseScheduler, EDMNoiseScheduler, ExpNoiseScheduler,
                        FlowNoiseScheduler, KarrasVENoiseScheduler, LinearNoiseScheduler, SqrtNoiseScheduler)
from .transforms import (DirectPredictionTransform, EpsilonPredictionTransform, FlowMatchPredictionTransform,
                         KarrasPredictionTransform, MinSNR, ScheduleWeighting, VPredictionTransform)

_LOGNORMAL = {"pixel": (-1.2, 1.2), "latent": (-0.4, 1.0)}


def _weighting(min_snr_gamma):
    return ScheduleWeighting() if min_snr_gamma is None else MinSNR(min_snr_gamma)


_PRED = {"epsilon": EpsilonPredictionTransform, "eps": EpsilonPredictionTransform, "v": VPredictionTransform,
         "direct": DirectPredictionTransform, "x0": DirectPredictionTransform}


@dataclass(frozen=True)
class EDM:
    sigma_min: float = 0.002
    sigma_max: float = 80.0
    rho: float = 7.0
    sigma_data: float = 0.5
    regime: Optional[str] = None
    P_mean: Optional[float] = None
    P_std: Optional[float] = None
    min_snr_gamma: Optional[float] = None

    def __post_init__(self):
        if self.regime not in (None, "pixel", "latent"):
            raise ValueError(f"EDM's regime is 'pixel' or 'latent', got {self.regime!r}")

    def lognormal(self):
        if self.P_mean is not None and self.P_std is not None:
            return self.P_mean, self.P_std
        if self.regime is None:
            raise ValueError("EDM draws training sigmas for one space: set regime='pixel' (-1.2, 1.2), "
                             "regime='latent' (-0.4, 1.0), or both P_mean and P_std")
        m, s = _LOGNORMAL[self.regime]
        return (m if self.P_mean is None else self.P_mean, s if self.P_std is None else self.P_std)

    def __call__(self) -> Process:
        m, s = self.lognormal()
        return Process(
            schedule=EDMNoiseScheduler(self.sigma_min, self.sigma_max, self.sigma_data, m, s),
            prediction=KarrasPredictionTransform(self.sigma_data),
            weighting=_weighting(self.min_snr_gamma),
            sampling=KarrasVENoiseScheduler(self.sigma_min, self.sigma_max, self.rho, self.sigma_data))


@dataclass(frozen=True)
class Karras:
    """Karras rho grid for training and sampling alike, EDM preconditioning."""
    sigma_min: float = 0.002
    sigma_max: float = 80.0
    rho: float = 7.0
    sigma_data: float = 0.5

    def __call__(self) -> Process:
        sched = KarrasVENoiseScheduler(self.sigma_min, self.sigma_max, self.rho, self.sigma_data)
        return Process(sched, KarrasPredictionTransform(self.sigma_data), ScheduleWeighting(), sched)


@dataclass(frozen=True)
class Cosine:
    timesteps: int = 1000
    prediction: str = "epsilon"
    min_snr_gamma: Optional[float] = None

    def __call__(self) -> Process:
        return Process(CosineNoiseScheduler(self.timesteps), _PRED[self.prediction](), _weighting(self.min_snr_gamma))


@dataclass(frozen=True)
class CosineContinuous:
    prediction: str = "v"
    min_snr_gamma: Optional[float] = None

    def __call__(self) -> Process:
        return Process(CosineContinuousNoiseScheduler(), _PRED[self.prediction](), _weighting(self.min_snr_gamma))


@dataclass(frozen=True)
class Linear:
    timesteps: int = 1000
    beta_start: float = 1e-4
    beta_end: float = 0.02
    prediction: str = "epsilon"

    def __call__(self) -> Process:
        return Process(LinearNoiseScheduler(self.timesteps, self.beta_start, self.beta_end), _PRED[self.prediction]())


@dataclass(frozen=True)
class Exp:
    sigma_min: float = 0.002
    sigma_max: float = 80.0
    sigma_data: float = 0.5

    def __call__(self) -> Process:
        sched = ExpNoiseScheduler(self.sigma_min, self.sigma_max, self.sigma_data)
        return Process(sched, KarrasPredictionTransform(self.sigma_data), ScheduleWeighting(), sched)


@dataclass(frozen=True)
class Sqrt:
    sigma_min: float = 0.002
    sigma_max: float = 80.0
    sigma_data: float = 0.5

    def __call__(self) -> Process:
        sched = SqrtNoiseScheduler(self.sigma_min, self.sigma_max, self.sigma_data)
        return Process(sched, KarrasPredictionTransform(self.sigma_data), ScheduleWeighting(), sched)


@dataclass(frozen=True)
class Flow:
    """Rectified flow / flow matching with a velocity target."""
    shift: float = 1.0
    logit_normal: bool = False

    def __call__(self) -> Process:
        sched = FlowNoiseScheduler(self.shift, self.logit_normal)
        return Process(sched, FlowMatchPredictionTransform(), ScheduleWeighting(), FlowNoiseScheduler(self.shift))


@dataclass(frozen=True)
class ResolutionShift:
    """Flow with the SD3-style resolution-dependent time shift sqrt(pixels / base_pixels)."""
    pixels: int = 1024 * 1024
    base_pixels: int = 256 * 256
    logit_normal: bool = True

    def __call__(self) -> Process:
        return Flow(shift=(self.pixels / self.base_pixels) ** 0.5, logit_normal=self.logit_normal)()


@dataclass(frozen=True)
class JiT:
    """"Just image Transformers": the rectified-flow path with the network predicting the clean image (x-prediction) and the
    loss taken on the implied velocity, which keeps a plain ViT on raw pixels well-conditioned at every noise level."""
    shift: float = 1.0
    logit_normal: bool = True

    def __call__(self) -> Process:
        sched = FlowNoiseScheduler(self.shift, self.logit_normal)
        return Process(sched, DirectPredictionTransform(), ScheduleWeighting(), FlowNoiseScheduler(self.shift))


@dataclass(frozen=True)
class MeanFlow:
    """The flow path for average-velocity training: the process is ``Flow``'s; the objective to pair it with is
    ``dew_b200.objectives.few_step.MeanFlowObjective`` (the network takes the interval's start ``r`` beside ``t``)."""
    flow_ratio: float = 0.5
    shift: float = 1.0
    objective: str = "MeanFlowObjective"

    def __call__(self) -> Process:
        return Flow(shift=self.shift)()


@dataclass(frozen=True)
class Shortcut:
    """The flow path for shortcut models (step size as an input): pair with ``few_step.ShortcutObjective``."""
    max_log2_steps: int = 7
    shift: float = 1.0
    objective: str = "ShortcutObjective"

    def __call__(self) -> Process:
        return Flow(shift=self.shift)()
