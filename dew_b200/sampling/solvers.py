"""Solvers: each takes one step of the reverse process across ``[t, t_next]``.

Protocol (reference: docs/design/api.md:213-227; src/dew/sampling/solvers/*.py):
``init(x, times, process, *, key) -> state`` and
``step(x, t, t_next, denoised, eps, state, key, process, denoise) -> (x, state)``.
``denoised`` / ``eps`` are the model's clean and noise estimates at ``(x, t)``; ``denoise(x, t)`` re-evaluates
the (guided) model for multi-stage methods.  Everything is written in (alpha, sigma) rates so one solver serves
variance-exploding, variance-preserving and flow schedules.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, List, Tuple

import torch

from ..diffusion.schedules import GeneralizedNoiseScheduler, expand
from ..utils import keys as K


def _rates(process, t, x):
    return process.rates(t, like=x)


def _noise(key, x):
    return K.normal(key, x.shape).to(x.device, x.dtype)


def _euler(x, denoised, source, target):
    """DDIM-form Euler step alpha_s x0 + sigma_s eps (no cancellation; lands on x0 at sigma 0)."""
    (a_t, s_t), (a_s, s_s) = source, target
    eps = (x - a_t * denoised) / s_t.clamp_min(1e-20)
    return a_s * denoised + s_s * eps


def _sigma_schedule(name, process) -> GeneralizedNoiseScheduler:
    sched = process.sampler_schedule()
    if not isinstance(sched, GeneralizedNoiseScheduler):
        raise TypeError(f"{name} integrates in sigma and needs a variance-exploding schedule, got {type(sched).__name__}")
    return sched


class Solver:
    def init(self, x, times, process, *, key):
        return ()

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        raise NotImplementedError


@dataclass
class Euler(Solver):
    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        return _euler(x, denoised, _rates(process, t, x), _rates(process, t_next, x)), state


@dataclass
class DDIM(Solver):
    """DDIM with stochasticity ``eta`` (eta = 0 is the deterministic Euler form)."""
    eta: float = 0.0

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        (a_t, s_t), (a_s, s_s) = _rates(process, t, x), _rates(process, t_next, x)
        if self.eta == 0.0:
            return a_s * denoised + s_s * eps, state
        # variance of the ancestral kernel in the (alpha, sigma) parameterisation
        ratio = (a_t / a_s.clamp_min(1e-20))
        var = (s_s ** 2 / s_t.clamp_min(1e-20) ** 2) * (s_t ** 2 - (ratio * s_s) ** 2).clamp_min(0)
        std = self.eta * torch.sqrt(var)
        det = torch.sqrt((s_s ** 2 - std ** 2).clamp_min(0))
        return a_s * denoised + det * eps + std * _noise(key, x), state


@dataclass
class DDPM(Solver):
    """Ancestral sampling from the DDPM posterior q(x_s | x_t, x_0)."""

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        return DDIM(eta=1.0).step(x, t, t_next, denoised, eps, state, key, process, denoise)


@dataclass
class EulerAncestral(Solver):
    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        _sigma_schedule("EulerAncestral", process)
        _, s_t = _rates(process, t, x)
        _, s_s = _rates(process, t_next, x)
        up = torch.minimum(s_s, torch.sqrt((s_s ** 2 * (s_t ** 2 - s_s ** 2) / s_t ** 2).clamp_min(0)))
        down = torch.sqrt((s_s ** 2 - up ** 2).clamp_min(0))
        d = (x - denoised) / s_t
        return x + d * (down - s_t) + _noise(key, x) * up, state


@dataclass
class Heun(Solver):
    """Karras et al. 2022 Algorithm 2 (with optional churn); the step to sigma = 0 is the Euler step."""
    s_churn: float = 0.0
    s_tmin: float = 0.0
    s_tmax: float = float("inf")
    s_noise: float = 1.0

    def init(self, x, times, process, *, key):
        if not self.s_churn:
            return ()
        sched = _sigma_schedule("Heun's churn", process)
        gamma = min(self.s_churn / (len(times) - 1), math.sqrt(2) - 1)
        sig = sched.sigmas(torch.as_tensor(times[:-1], dtype=torch.float32))
        churned = (sig >= self.s_tmin) & (sig <= self.s_tmax)
        top = sched.sigma_range()[1]
        if bool((churned & (sig * (1 + gamma) > top * (1 + 1e-6))).any()):
            raise ValueError(f"the churn raises sigma past the schedule's top {top}; keep s_tmax below {top / (1 + gamma):.4g}")
        return gamma

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        if self.s_churn:
            sched = _sigma_schedule("Heun's churn", process)
            sigma = sched.sigmas(t)
            gamma = torch.where((sigma >= self.s_tmin) & (sigma <= self.s_tmax),
                                torch.full_like(sigma, float(state)), torch.zeros_like(sigma))
            spread = sigma * torch.sqrt(gamma * (2 + gamma)) * self.s_noise
            x = x + expand(spread.to(x.device), x) * _noise(key, x)
            t = sched.t_of_sigma(sigma * (1 + gamma))
            denoised, _ = denoise(x, t)
        src, tgt = _rates(process, t, x), _rates(process, t_next, x)
        (a_t, s_t), (a_s, s_s) = src, tgt
        x_euler = _euler(x, denoised, src, tgt)
        if bool((s_s == 0).all()):
            return x_euler, state
        dt = s_s - s_t
        coeff = (a_t * s_s - a_s * s_t) / torch.where(dt == 0, torch.ones_like(dt), dt)
        d0 = (x - coeff * denoised) / s_t
        den_next, _ = denoise(x_euler, t_next)
        safe = torch.where(s_s > 0, s_s, torch.ones_like(s_s))
        d1 = (x_euler - coeff * den_next) / safe
        return torch.where(s_s > 0, x + 0.5 * (d0 + d1) * dt, x_euler), state


@dataclass
class RK4(Solver):
    """Classical Runge-Kutta on the probability-flow ODE in sigma (variance-exploding schedules)."""

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        sched = _sigma_schedule("RK4", process)
        _, s_t = _rates(process, t, x)
        _, s_s = _rates(process, t_next, x)
        if bool((s_s == 0).all()):
            return denoised, state
        h = s_s - s_t
        t_mid = sched.t_of_sigma((sched.sigmas(t) + sched.sigmas(t_next)) / 2)
        s_m = expand(((sched.sigmas(t) + sched.sigmas(t_next)) / 2).to(x.device), x)

        def f(xx, tt, ss, den=None):
            d = denoise(xx, tt)[0] if den is None else den
            return (xx - d) / ss
        k1 = f(x, t, s_t, denoised)
        k2 = f(x + 0.5 * h * k1, t_mid, s_m)
        k3 = f(x + 0.5 * h * k2, t_mid, s_m)
        k4 = f(x + h * k3, t_next, s_s)
        return x + h / 6 * (k1 + 2 * k2 + 2 * k3 + k4), state


@dataclass
class KDPM2(Solver):
    """k-diffusion DPM2: midpoint method in log-sigma."""

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        sched = _sigma_schedule("KDPM2", process)
        _, s_t = _rates(process, t, x)
        _, s_s = _rates(process, t_next, x)
        d = (x - denoised) / s_t
        if bool((s_s == 0).all()):
            return x + d * (s_s - s_t), state
        sig_mid = torch.exp((torch.log(sched.sigmas(t)) + torch.log(sched.sigmas(t_next))) / 2)
        s_m = expand(sig_mid.to(x.device), x)
        x_mid = x + d * (s_m - s_t)
        den_mid, _ = denoise(x_mid, sched.t_of_sigma(sig_mid))
        d_mid = (x_mid - den_mid) / s_m
        return x + d_mid * (s_s - s_t), state


def _lambda(a, s):
    return torch.log(a.clamp_min(1e-20)) - torch.log(s.clamp_min(1e-20))


@dataclass
class DPMSolverMultistep(Solver):
    """DPM-Solver++ (2M by default) in data-prediction form; ``order`` 1-3; first/last steps lower order."""
    order: int = 2

    def init(self, x, times, process, *, key):
        return {"hist": [], "n": len(times) - 1, "i": 0}

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        (a_t, s_t), (a_s, s_s) = _rates(process, t, x), _rates(process, t_next, x)
        hist: List[Tuple[torch.Tensor, torch.Tensor]] = list(state["hist"])
        i, n = state["i"], state["n"]
        new_state = {"hist": ([(denoised, _lambda(a_t, s_t))] + hist)[: self.order], "n": n, "i": i + 1}
        if bool((s_s == 0).all()):
            return a_s * denoised, new_state
        lam_t, lam_s = _lambda(a_t, s_t), _lambda(a_s, s_s)
        h = lam_s - lam_t
        order = min(self.order, len(hist) + 1, n - i)  # lower order near the end
        phi = torch.expm1(-h)
        D = denoised
        if order >= 2 and hist:
            d1, lam1 = hist[0]
            r0 = (lam_t - lam1) / h
            D1 = (denoised - d1) / r0
            if order >= 3 and len(hist) >= 2:
                d2, lam2 = hist[1]
                r1 = (lam1 - lam2) / h
                D1_1 = (d1 - d2) / r1
                D1n = D1 + (r0 / (r0 + r1)) * (D1 - D1_1)
                D2 = (D1 - D1_1) / (r0 + r1)
                x_next = (s_s / s_t) * x - a_s * phi * D + a_s * (phi / h + 1) * D1n - a_s * ((phi + h) / h ** 2 - 0.5) * D2
                return x_next, new_state
            D = denoised + 0.5 * D1
        return (s_s / s_t) * x - a_s * phi * D, new_state


@dataclass
class MultiStepDPM(DPMSolverMultistep):
    """k-diffusion ``sample_dpmpp_2m`` naming for DPM-Solver++ 2M."""


@dataclass
class DPMSolverSinglestep(Solver):
    """DPM-Solver++ 2S: one intermediate evaluation at the log-SNR midpoint."""

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        (a_t, s_t), (a_s, s_s) = _rates(process, t, x), _rates(process, t_next, x)
        if bool((s_s == 0).all()):
            return a_s * denoised, state
        t_mid = (torch.as_tensor(t) + torch.as_tensor(t_next)) / 2
        a_m, s_m = _rates(process, t_mid, x)
        lam_t, lam_m, lam_s = _lambda(a_t, s_t), _lambda(a_m, s_m), _lambda(a_s, s_s)
        h, h1 = lam_s - lam_t, lam_m - lam_t
        x_m = (s_m / s_t) * x - a_m * torch.expm1(-h1) * denoised
        den_m, _ = denoise(x_m, t_mid)
        r = h1 / h
        D = denoised + (den_m - denoised) / (2 * r)
        return (s_s / s_t) * x - a_s * torch.expm1(-h) * D, state


@dataclass
class DEIS(Solver):
    """Exponential integrator with Adams-Bashforth extrapolation of eps in log-SNR (t-AB-DEIS, order <= 3)."""
    order: int = 2

    def init(self, x, times, process, *, key):
        return {"hist": []}

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        (a_t, s_t), (a_s, s_s) = _rates(process, t, x), _rates(process, t_next, x)
        hist = list(state["hist"])
        lam_t = _lambda(a_t, s_t)
        new_state = {"hist": ([(eps, lam_t)] + hist)[: self.order]}
        if bool((s_s == 0).all()):
            return a_s * denoised, new_state
        lam_s = _lambda(a_s, s_s)
        h = lam_s - lam_t
        E = eps
        if self.order >= 2 and hist:
            e1, lam1 = hist[0]
            E = eps + 0.5 * h / (lam_t - lam1) * (eps - e1)
        return (a_s / a_t) * x - s_s * torch.expm1(h) * E, new_state


@dataclass
class UniPC(Solver):
    """UniPC-p predictor (B(h) = expm1) with a UniC corrector applied at the next evaluation, data prediction."""
    order: int = 2

    def init(self, x, times, process, *, key):
        return {"hist": [], "pending": None}

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        (a_t, s_t), (a_s, s_s) = _rates(process, t, x), _rates(process, t_next, x)
        hist = list(state["hist"])
        lam_t = _lambda(a_t, s_t)
        pending = state["pending"]
        if pending is not None:  # corrector: re-do the previous step with the now-known endpoint value
            x_prev, d_prev, lam_prev, (a_p, s_p) = pending
            h = lam_t - lam_prev
            phi = torch.expm1(-h)
            x = (s_t / s_p) * x_prev - a_t * phi * d_prev - a_t * phi * 0.5 * (denoised - d_prev)
        new_hist = ([(denoised, lam_t)] + hist)[: self.order]
        if bool((s_s == 0).all()):
            return a_s * denoised, {"hist": new_hist, "pending": None}
        lam_s = _lambda(a_s, s_s)
        h = lam_s - lam_t
        phi = torch.expm1(-h)
        D = denoised
        if self.order >= 2 and hist:
            d1, lam1 = hist[0]
            D = denoised + 0.5 * (denoised - d1) * (h / (lam_t - lam1))
        x_next = (s_s / s_t) * x - a_s * phi * D
        return x_next, {"hist": new_hist, "pending": (x, denoised, lam_t, (a_t, s_t))}


@dataclass
class LMS(Solver):
    """Linear multistep (Adams-Bashforth in sigma) over the derivative history, k-diffusion's ``sample_lms``."""
    order: int = 4

    def init(self, x, times, process, *, key):
        return {"hist": [], "sig": []}

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        sched = _sigma_schedule("LMS", process)
        _, s_t = _rates(process, t, x)
        _, s_s = _rates(process, t_next, x)
        d = (x - denoised) / s_t
        sig_t = float(sched.sigmas(torch.as_tensor(t).flatten()[0]))
        sig_s = float(sched.sigmas(torch.as_tensor(t_next).flatten()[0]))
        ds = ([d] + list(state["hist"]))[: self.order]
        sg = ([sig_t] + list(state["sig"]))[: self.order]
        k = len(ds)
        # integrate Lagrange basis polynomials over [sig_t, sig_s] with Gauss-Legendre quadrature (exact here)
        nodes, wts = _gauss_legendre(8)
        out = x
        for j in range(k):
            total = 0.0
            for u, w in zip(nodes, wts):
                tau = 0.5 * (sig_s - sig_t) * u + 0.5 * (sig_s + sig_t)
                prod = 1.0
                for m in range(k):
                    if m != j:
                        prod *= (tau - sg[m]) / (sg[j] - sg[m])
                total += w * prod
            out = out + ds[j] * (total * 0.5 * (sig_s - sig_t))
        return out, {"hist": ds, "sig": sg}


def _gauss_legendre(n):
    import numpy as np
    x, w = np.polynomial.legendre.leggauss(n)
    return x.tolist(), w.tolist()


@dataclass
class PNDM(Solver):
    """Pseudo linear multistep (PLMS): Adams-Bashforth on eps, transferred with the DDIM map."""

    def init(self, x, times, process, *, key):
        return {"hist": []}

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        (a_t, s_t), (a_s, s_s) = _rates(process, t, x), _rates(process, t_next, x)
        h = list(state["hist"])
        if len(h) == 0:
            e = eps
        elif len(h) == 1:
            e = (3 * eps - h[0]) / 2
        elif len(h) == 2:
            e = (23 * eps - 16 * h[0] + 5 * h[1]) / 12
        else:
            e = (55 * eps - 59 * h[0] + 37 * h[1] - 9 * h[2]) / 24
        x0 = (x - s_t * e) / a_t.clamp_min(1e-20)
        return a_s * x0 + s_s * e, {"hist": ([eps] + h)[:3]}


@dataclass
class DPMSolverSDE(Solver):
    """DPM-Solver++ SDE (first order, data prediction) with noise of the exact reverse-SDE variance."""
    eta: float = 1.0

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        (a_t, s_t), (a_s, s_s) = _rates(process, t, x), _rates(process, t_next, x)
        if bool((s_s == 0).all()):
            return a_s * denoised, state
        h = _lambda(a_s, s_s) - _lambda(a_t, s_t)
        eh = self.eta * h
        x_next = (s_s / s_t) * torch.exp(-eh) * x + a_s * (-torch.expm1(-h - eh)) * denoised
        return x_next + s_s * torch.sqrt((-torch.expm1(-2 * eh)).clamp_min(0)) * _noise(key, x), state


@dataclass
class Consistency(Solver):
    """Multistep consistency sampling: jump to x_0, re-noise to the next level."""

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        a_s, s_s = _rates(process, t_next, x)
        return a_s * denoised + s_s * _noise(key, x), state


@dataclass
class TCD(Solver):
    """Trajectory consistency distillation sampling with stochasticity ``gamma``."""
    gamma: float = 0.3

    def step(self, x, t, t_next, denoised, eps, state, key, process, denoise):
        t_mid = (1 - self.gamma) * torch.as_tensor(t_next)
        a_m, s_m = _rates(process, t_mid, x)
        a_s, s_s = _rates(process, t_next, x)
        x_m = a_m * denoised + s_m * eps
        if self.gamma == 0 or bool((s_s == 0).all()):
            return a_s * denoised + s_s * eps, state
        ratio = a_s / a_m.clamp_min(1e-20)
        return ratio * x_m + torch.sqrt((s_s ** 2 - (ratio * s_m) ** 2).clamp_min(0)) * _noise(key, x), state


SOLVERS = {c.__name__: c for c in (Euler, EulerAncestral, Heun, RK4, KDPM2, MultiStepDPM, LMS, DDPM, DDIM, PNDM,
                                    Consistency, TCD, DPMSolverMultistep, DPMSolverSinglestep, DEIS, UniPC, DPMSolverSDE)}
