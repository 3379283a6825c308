"""Stochastic rectified-flow transitions with Gaussian likelihoods (the sampler Flow-GRPO scores).

The reverse ODE of a rectified flow is turned into an SDE with the same marginals and the diffusion coefficient
``a sqrt(sigma / (1 - sigma))`` (``a`` = ``noise_level``, arXiv 2505.05470 eq. 8-9).  One Euler-Maruyama step from noise
rate ``sigma`` to ``sigma_next`` is an isotropic Gaussian whose mean and variance are closed forms of the state and the
model's velocity, so a trajectory can be sampled once and each of its transitions rescored later under other weights.

Reference: src/dew/sampling/flow.py (``GaussianTransition`` :36, ``flow_transition`` :362, ``FlowSDE`` :398, ``FlowTrajectory``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..utils import keys as K
from .solvers import Solver
from .walks import sample


def _rows(v: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    return v.reshape(-1, *([1] * (like.dim() - 1)))


@dataclass
class GaussianTransition:
    """Isotropic Gaussian over the next state with one variance per row.  A zero variance is a deterministic transition:
    sampling returns the mean and the density is NaN (a point mass has none)."""
    mean: torch.Tensor
    variance: torch.Tensor          # [B]

    @property
    def stochastic(self) -> torch.Tensor:
        return self.variance > 0

    def sample(self, key) -> torch.Tensor:
        if not bool((self.variance > 0).any()):
            return self.mean
        z = K.normal(key, self.mean.shape).to(self.mean.device, self.mean.dtype)
        return self.mean + _rows(self.variance.clamp_min(0).sqrt(), self.mean) * z

    def log_prob(self, value: torch.Tensor) -> torch.Tensor:
        """Joint log density of ``value`` per row, summed over the sample dimensions."""
        if value.shape != self.mean.shape:
            raise ValueError("a transition density scores one next state per mean")
        var = torch.where(self.variance > 0, self.variance, torch.ones_like(self.variance))
        d = math.prod(value.shape[1:])
        sq = ((value.to(self.mean.dtype) - self.mean) ** 2).reshape(value.shape[0], -1).sum(1)
        lp = -0.5 * (sq / var + d * (math.log(2 * math.pi) + torch.log(var)))
        return torch.where(self.variance > 0, lp, torch.full_like(lp, float("nan")))

    def kl(self, reference_mean: torch.Tensor) -> torch.Tensor:
        """KL(this || a transition with the same variance and ``reference_mean``) per row: ``|mu - mu_ref|^2 / (2 var)``."""
        sq = ((self.mean - reference_mean.to(self.mean.dtype)) ** 2).reshape(self.mean.shape[0], -1).sum(1)
        var = torch.where(self.variance > 0, self.variance, torch.ones_like(self.variance))
        return torch.where(self.variance > 0, sq / (2 * var), torch.zeros_like(sq))


def flow_transition(x: torch.Tensor, velocity: torch.Tensor, sigma, sigma_next, *, noise_level: float = 0.7) -> GaussianTransition:
    """Euler-Maruyama over the noise rate, ``0 <= sigma_next <= sigma <= 1``; ``velocity = noise - clean``.

    With ``c = a^2 / (2 (1 - sigma))`` (at ``sigma = 1`` the denominator uses ``sigma_next``, as the Flow-GRPO code does) and
    ``dt = sigma_next - sigma``:  mean ``= x (1 + c dt) + v (1 + c (1 - sigma)) dt``,  variance ``= a^2 sigma / (1 - sigma) (-dt)``.
    Rates outside the domain give NaN transitions; zero noise or a zero step is deterministic."""
    if not math.isfinite(noise_level) or noise_level < 0:
        raise ValueError("noise_level must be finite and non-negative")
    if x.dim() < 2 or velocity.shape != x.shape:
        raise ValueError("x and velocity must share a [batch, ...] sample shape")
    dt_ = torch.float64 if x.dtype == torch.float64 else torch.float32
    x, velocity = x.to(dt_), velocity.to(dt_)
    B = x.shape[0]
    s = torch.as_tensor(sigma, dtype=dt_, device=x.device).expand(B)
    sn = torch.as_tensor(sigma_next, dtype=dt_, device=x.device).expand(B)
    dt = sn - s
    valid = (sn >= 0) & (s <= 1) & (dt <= 0)
    denom = torch.where(dt == 0, torch.ones_like(s), 1 - torch.where(s == 1, sn, s))
    c = noise_level ** 2 / (2 * denom)
    mean = x * _rows(1 + c * dt, x) + velocity * _rows((1 + c * (1 - s)) * dt, x)
    var = noise_level ** 2 * s / denom * (-dt)
    nan = torch.full_like(var, float("nan"))
    return GaussianTransition(torch.where(_rows(valid, x), mean, torch.full_like(mean, float("nan"))), torch.where(valid, var, nan))


@dataclass
class FlowTrajectory:
    """``states [B, points, ...]``, ``times [points]``, ``log_probs`` and ``stochastic`` ``[B, points - 1]``."""
    states: torch.Tensor
    times: torch.Tensor
    log_probs: torch.Tensor
    stochastic: torch.Tensor

    @property
    def samples(self) -> torch.Tensor:
        return self.states[:, -1]


@dataclass
class FlowSDE(Solver):
    """Solver for ``sample`` that draws every step from ``flow_transition``; its state is (log density of the draw, whether
    the step was stochastic), per row."""
    noise_level: float = 0.7

    def validate(self, process) -> None:
        from ..diffusion.schedules import FlowNoiseScheduler as RectifiedFlow
        if not isinstance(process.sampler_schedule(), RectifiedFlow):
            raise ValueError("FlowSDE requires a rectified-flow schedule")

    def init(self, x, times, process, *, key):
        self.validate(process)
        return torch.full((x.shape[0],), float("nan"), device=x.device), torch.zeros(x.shape[0], dtype=torch.bool, device=x.device)

    def transition(self, x, t, t_next, denoised, eps, process) -> GaussianTransition:
        sched = process.sampler_schedule()
        sigma = sched.rates(t)[1].reshape(-1)
        following = sched.rates(t_next)[1].reshape(-1)
        return flow_transition(x, eps - denoised, sigma.to(x.device), following.to(x.device), noise_level=self.noise_level)

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        tr = self.transition(x, t, t_next, denoised, eps, process)
        nxt = tr.sample(key)
        return nxt, (tr.log_prob(nxt), tr.stochastic)

    def trajectory(self, denoise, x_T: torch.Tensor, steps: int, *, guidance=None, key=0) -> FlowTrajectory:
        """``sample`` with this solver, recording every state with its log density; ``steps`` counts grid points (both ends),
        so ten transitions take ``steps=11``.  The last transition already lands on the sample (a rectified flow's clean
        prediction at time 0 is its state), so no final denoise is taken."""
        if steps < 2:
            raise ValueError("a trajectory needs at least two time points")
        if guidance is not None and getattr(guidance, "momentum", 0):
            raise ValueError("a flow trajectory's transitions are rescored one at a time, so its guidance carries nothing "
                             "between steps; APG's momentum does")
        x_T = x_T.float() if x_T.dtype in (torch.bfloat16, torch.float16) else x_T
        _, rec = sample(denoise, x_T, steps - 1, solver=self, guidance=guidance, key=key, final_denoise=False,
                        record=lambda following, state, denoised: (following, state[0], state[1]))
        states = torch.stack([x_T] + [r[0] for r in rec], 1)
        return FlowTrajectory(states, denoise.process.times(steps - 1), torch.stack([r[1] for r in rec], 1), torch.stack([r[2] for r in rec], 1))

    def rescore(self, denoise, trajectory: FlowTrajectory, index: int, *, guidance=None) -> GaussianTransition:
        """The transition ``index -> index + 1`` of a recorded trajectory under ``denoise`` (differentiable: no ``no_grad``)."""
        x = trajectory.states[:, index]
        B = x.shape[0]
        t = torch.full((B,), float(trajectory.times[index]), device=x.device)
        tn = torch.full((B,), float(trajectory.times[index + 1]), device=x.device)
        call = guidance.wrap(denoise, None) if guidance is not None else denoise
        denoised, eps = call(x, t)
        return self.transition(x, t, tn, denoised, eps, denoise.process)
