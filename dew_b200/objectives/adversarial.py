"""Adversarial diffusion distillation (LADD, with ADD's distillation term and R1 penalty).

A few-step student is trained against a projected discriminator built on the frozen teacher: the student's clean
prediction and a real sample are both noised again, the teacher reads each, and independent heads on the teacher's token
sequences after chosen blocks score them with the hinge loss (Sauer et al. 2024; heads after StyleGAN-T's ``DiscHead`` with
2-D convolutions over the token grid, conditioned by projection on the noise level).  ADD (Sauer et al. 2023) adds the R1
penalty on each head's input (gamma 1e-5) and a distillation term that pulls the student's prediction toward the teacher's
denoising of it (lambda 2.5).  Student and heads are trained by ONE backward: the generator term reads the heads through
detached weights and the discriminator term reads detached features, so each loss reaches only its own parameters.

Reference: src/dew/objectives/diffusion/adversarial.py (``Head`` :133, ``Heads`` :159, ``hinge_discriminator`` :174,
``hinge_generator`` :181, ``r1_penalty`` :190, ``AdversarialDistillationObjective`` :203-362).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn.utils.parametrizations import spectral_norm

from ..diffusion.schedules import expand
from ..nn.layers import sinusoidal
from .base import Aux, Ratio, Step
from .diffusion import DiffusionObjective


class Head(nn.Module):
    """One discriminator head over a ``[B, N, W]`` token sequence on a square grid: spectral-normalised 1x1 and 3x3 (circular
    residual) convolutions, then a projection on the condition vector -> one logit per token."""

    def __init__(self, width: int, channels: int = 64, condition: int = 64):
        super().__init__()
        self.inp = spectral_norm(nn.Conv2d(width, channels, 1))
        self.mix = spectral_norm(nn.Conv2d(channels, channels, 3, padding=1, padding_mode="circular"))
        self.out = spectral_norm(nn.Conv2d(channels, condition, 1))
        self.cmap = nn.Linear(condition, condition)
        self.norm1, self.norm2 = nn.GroupNorm(8, channels), nn.GroupNorm(8, channels)

    def forward(self, tokens: torch.Tensor, condition: torch.Tensor) -> torch.Tensor:
        B, N, W = tokens.shape
        side = math.isqrt(N)
        if side * side != N:
            raise ValueError(f"a discriminator head needs a square token grid, not {N} tokens")
        x = tokens.float().reshape(B, side, side, W).permute(0, 3, 1, 2)
        x = F.leaky_relu(self.norm1(self.inp(x)), 0.2)
        x = (x + F.leaky_relu(self.norm2(self.mix(x)), 0.2)) / math.sqrt(2)
        x = self.out(x)                                                        # [B, C, s, s]
        c = self.cmap(condition.float())[:, :, None, None]
        return (x * c).sum(1).reshape(B, N) / math.sqrt(x.shape[1])


class Heads(nn.Module):
    def __init__(self, count: int, width: int, channels: int = 64, condition: int = 64):
        super().__init__()
        self.heads = nn.ModuleList([Head(width, channels, condition) for _ in range(count)])
        self.condition = condition

    def forward(self, features: Sequence[torch.Tensor], condition: torch.Tensor) -> List[torch.Tensor]:
        return [h(f, condition) for h, f in zip(self.heads, features)]


def hinge_discriminator(real: Sequence[torch.Tensor], fake: Sequence[torch.Tensor]) -> torch.Tensor:
    return sum(F.relu(1 - r).mean() + F.relu(1 + f).mean() for r, f in zip(real, fake))


def hinge_generator(fake: Sequence[torch.Tensor]) -> torch.Tensor:
    return -sum(f.mean() for f in fake)


def r1_penalty(heads: Heads, features: Sequence[torch.Tensor], condition: torch.Tensor) -> torch.Tensor:
    """Squared gradient norm of the summed real scores w.r.t. each head's input, mean over rows (differentiable)."""
    feats = [f.detach().requires_grad_(True) for f in features]
    total = sum(s.sum() for s in heads(feats, condition))
    grads = torch.autograd.grad(total, feats, create_graph=True)
    return sum(g.pow(2).reshape(g.shape[0], -1).sum(1).mean() for g in grads)


class _StudentWithHeads(nn.Module):
    def __init__(self, student: nn.Module, heads: Heads):
        super().__init__()
        self.backbone, self.discriminator = student, heads

    def forward(self, *args, **kwargs):
        return self.backbone(*args, **kwargs)


class AdversarialDistillationObjective(DiffusionObjective):
    """``model``: the few-step student; ``teacher``: a frozen denoiser over the same process and inputs whose submodules
    ``layers`` (each yielding ``[B, N, width]`` tokens) feed the discriminator heads.  Each row draws its student time from
    ``student_times`` (the few-step grid the student is sampled on) and a fresh re-noising time from the process's schedule.

    loss = hinge_G(student) + ``distill_weight`` * w(t') |x_student - teacher(renoised x_student)|^2 / 2
         + hinge_D(heads) + ``r1_gamma`` * R1(heads on real features)
    """

    def __init__(self, model: nn.Module, process=None, inputs=None, *, teacher: nn.Module, layers: Sequence[str], width: int,
                 student_times: Sequence[float] = (1.0, 0.75, 0.5, 0.25), distill_weight: float = 2.5, r1_gamma: float = 1e-5,
                 head_channels: int = 64, **kw):
        kw.setdefault("guidance", None)
        heads = Heads(len(layers), width, head_channels, head_channels)
        p = next(model.parameters(), None)
        if p is not None:
            heads = heads.to(p.device)
        super().__init__(_StudentWithHeads(model, heads), process, inputs, **kw)
        self.teacher = teacher.requires_grad_(False).eval()
        self.layers = tuple(layers)
        if not self.layers:
            raise ValueError("the discriminator reads the teacher after at least one block")
        self.student_times = tuple(float(t) for t in student_times)
        self.distill_weight, self.r1_gamma = float(distill_weight), float(r1_gamma)
        self._kept: List[torch.Tensor] = []
        for name in self.layers:
            self.teacher.get_submodule(name).register_forward_hook(lambda m, a, out: self._kept.append(out[0] if isinstance(out, tuple) else out))

    # -- pieces
    def _teacher(self, x_t, t, conditions) -> Tuple[torch.Tensor, List[torch.Tensor]]:
        """The teacher's clean prediction of ``x_t`` and its token features at ``layers`` (gradients flow to ``x_t``)."""
        self._kept = []
        den = self.process.denoiser(self.teacher, None, conditions)
        clean, _ = den(x_t, t)
        feats, self._kept = self._kept, []
        if len(feats) != len(self.layers):
            raise RuntimeError("a discriminator layer did not run in the teacher's call")
        return clean, feats

    def _condition(self, t: torch.Tensor) -> torch.Tensor:
        return sinusoidal(self.process.schedule.model_time(t), self.model.discriminator.condition)

    def loss(self, variables, batch, step: Step):
        x0 = batch[self.inputs.sample.key]
        if self.autoencoder is not None:
            with torch.no_grad():
                x0 = self.autoencoder.encode(x0)
        x0 = x0.float()
        rows, dev = x0.shape[0], x0.device
        sched, pred = self.process.schedule, self.process.prediction
        conditions = self._conditions(batch, step, rows, drop=False)
        # the student denoises a sample noised at one of its few-step times
        pick = (step.sample("student time", (), rows, kind="uniform") * len(self.student_times)).long().clamp_max(len(self.student_times) - 1)
        ts = torch.tensor(self.student_times)[pick].to(dev)
        x_ts, _, _ = pred.forward_diffusion(x0, step.sample("student noise", x0.shape[1:], rows).to(dev), self.process.rates(ts, like=x0))
        student = self.process.denoiser(self.model, variables, conditions)
        fake, _ = student(x_ts, ts)
        fake = fake.float()
        # both are noised again and read by the frozen teacher
        t2 = torch.stack([sched.sample_t(k, 1)[0] for k in step.row_keys("renoise time", rows)]).to(dev)
        rates2 = self.process.rates(t2, like=x0)
        n2 = step.sample("renoise", x0.shape[1:], rows).to(dev)
        fake_t, _, _ = pred.forward_diffusion(fake, n2, rates2)
        real_t, _, _ = pred.forward_diffusion(x0, n2, rates2)
        teacher_clean, fake_feats = self._teacher(fake_t, t2, conditions)
        with torch.no_grad():
            _, real_feats = self._teacher(real_t, t2, conditions)
        cond = self._condition(t2).to(dev)
        heads = self.model.discriminator
        from ..utils.trees import variables_for_call
        live = None
        if variables is not None:
            flat = variables_for_call(self.model, variables)
            live = {k[len("discriminator."):]: v for k, v in flat.items() if k.startswith("discriminator.")}
        score = (lambda f, params: torch.func.functional_call(heads, params, (f, cond))) if live is not None else (lambda f, params: heads(f, cond))
        # generator: the heads' weights are constants here (spectral norm's power iteration is not advanced)
        was = heads.training
        heads.eval()
        frozen = {k: v.detach() for k, v in live.items()} if live is not None else None
        if frozen is None:
            for p_ in heads.parameters():
                p_.requires_grad_(False)
        g_loss = hinge_generator(score(fake_feats, frozen))
        if frozen is None:
            for p_ in heads.parameters():
                p_.requires_grad_(True)
        heads.train(was)
        # distillation toward the teacher's denoising of the re-noised prediction
        w = expand(self.process.weight(t2).to(dev), fake)
        distill = (0.5 * (fake - teacher_clean.detach().float()) ** 2 * w).reshape(rows, -1).mean(1).mean()
        # discriminator: features are constants here
        d_real = score([f.detach() for f in real_feats], live)
        d_fake = score([f.detach() for f in fake_feats], live)
        d_loss = hinge_discriminator(d_real, d_fake)
        r1 = r1_penalty(heads, real_feats, cond) if self.r1_gamma > 0 else torch.zeros((), device=dev)
        total = g_loss + self.distill_weight * distill + d_loss + self.r1_gamma * r1
        one = torch.ones((), device=dev)
        mass = torch.tensor(float(rows), device=dev)
        metrics = {"generator": Ratio(g_loss.detach(), one), "discriminator": Ratio(d_loss.detach(), one),
                   "distillation": Ratio(distill.detach(), one), "r1": Ratio(r1.detach(), one),
                   "real_score": Ratio(sum(s.mean() for s in d_real).detach() / len(d_real), one),
                   "fake_score": Ratio(sum(s.mean() for s in d_fake).detach() / len(d_fake), one)}
        return Ratio(total * mass, mass), Aux(metrics=metrics)

    def generate(self, variables, shape, *, key=0, conditions=None, steps=None, solver=None, guidance="default"):
        """Few-step sampling on the student's own time grid (``student_times`` then 0)."""
        from ..sampling import Euler, sample
        from ..utils import keys as K
        den = self.process.denoiser(self.model, variables, conditions or {})
        dev = next(self.model.parameters()).device
        x_T = self.process.noise(K.fold_in(K.key(key), "prior"), shape).to(dev)
        x = sample(den, x_T, times=list(self.student_times) + [0.0], solver=solver or Euler(), key=key, final_denoise=False)
        return self.autoencoder.decode(x) if self.autoencoder is not None else x
