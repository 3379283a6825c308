"""REPA-E: the autoencoder trained together with the latent diffusion model through representation alignment.

One loss makes the reference's updates at once by stopping each gradient where that recipe freezes a part
(Leng et al. 2025, "REPA-E: Unlocking VAE for End-to-End Tuning with Latent Diffusion Transformers"):

* the autoencoder: L1 reconstruction + ``kl_weight`` KL + ``vae_align`` x the alignment loss of ITS latent, read through the
  diffusion model with that model's weights held constant (the gradient reaches the encoder through the latent only);
* the diffusion model: the denoising loss and ``alignment.weight / 2`` x the alignment loss on the DETACHED latent, so the
  denoising loss cannot collapse the latent space (the failure REPA-E names).

Both read the same latent draw, times and noise.  The reference's PatchGAN / LPIPS terms of the autoencoder's own loss need
pretrained networks and are left to the caller (``extra_vae_loss(reconstruction, images)``).

Reference: src/dew/objectives/diffusion/end_to_end.py; src/dew/objectives/diffusion/alignment.py.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..diffusion.schedules import expand
from .base import Aux, Ratio, Step
from .diffusion import DiffusionObjective
from .diffusion_extras import Alignment, AlignedModel, Projector


class _Joint(nn.Module):
    def __init__(self, denoiser: AlignedModel, autoencoder: nn.Module):
        super().__init__()
        self.denoiser, self.autoencoder = denoiser, autoencoder

    def forward(self, *args, **kwargs):
        return self.denoiser(*args, **kwargs)


class EndToEndObjective(DiffusionObjective):
    def __init__(self, model: nn.Module, autoencoder: nn.Module, process=None, inputs=None, *, alignment: Alignment, hidden_features: int,
                 encoder_features: int, vae_align: float = 1.5, kl_weight: float = 1e-6,
                 extra_vae_loss: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None, **kw):
        proj = Projector(alignment.projector, hidden_features, encoder_features, alignment.width, alignment.kernel_size)
        p = next(model.parameters(), None)
        if p is not None:
            proj = proj.to(p.device)
        super().__init__(_Joint(AlignedModel(model, proj, alignment.layer), autoencoder), process, inputs, autoencoder=None, **kw)
        self.alignment, self.vae_align, self.kl_weight, self.extra_vae_loss = alignment, float(vae_align), float(kl_weight), extra_vae_loss
        self.vae = autoencoder

    def _align(self, hidden, targets, frozen: bool):
        proj = self.model.denoiser.alignment_projector
        if frozen:
            params = {k: v.detach() for k, v in proj.named_parameters()}
            projected = torch.func.functional_call(proj, params, (hidden.float(),))
        else:
            projected = proj(hidden.float())
        return -F.cosine_similarity(projected.float(), targets, dim=-1).mean(1)          # [B]

    def _denoise(self, latent, t, noise, frozen: bool):
        """Raw output, target, weight and the aligned layer's hidden tokens for one latent (weights constant when ``frozen``)."""
        sched, pred = self.process.schedule, self.process.prediction
        rates = self.process.rates(t, like=latent)
        x_t, c_in, target = pred.forward_diffusion(latent, noise, rates)
        den = self.model.denoiser
        if frozen:
            params = {k: v.detach() for k, v in den.named_parameters()}
            raw = torch.func.functional_call(den, params, (x_t * c_in, sched.model_time(t), {}))
        else:
            raw = den(x_t * c_in, sched.model_time(t), {})
        hidden, den.hidden = den.hidden, None
        out = pred.pred_transform(x_t, raw.float(), rates, t)
        return out, target, hidden

    def loss(self, variables, batch, step: Step):
        images = batch[self.inputs.sample.key].float()
        rows, dev = images.shape[0], images.device
        mean, logvar = self.vae.moments(images)
        logvar = logvar.clamp(-30, 20)
        z = mean + torch.exp(0.5 * logvar) * step.sample("latent", mean.shape[1:], rows).to(dev)
        latent = (z * self.vae.scale).permute(0, 2, 3, 1)
        recon = self.vae.decode(latent)
        kl = 0.5 * (mean ** 2 + logvar.exp() - 1 - logvar).reshape(rows, -1).mean(1)
        vae_own = (recon - images).abs().reshape(rows, -1).mean(1) + self.kl_weight * kl
        if self.extra_vae_loss is not None:
            vae_own = vae_own + self.extra_vae_loss(recon, images)
        sched = self.process.schedule
        t = torch.stack([sched.sample_t(k, 1)[0] for k in step.row_keys("time", rows)]).to(dev)
        noise = step.sample("noise", latent.shape[1:], rows).to(dev)
        targets = self.alignment.targets(images)
        # the autoencoder's alignment term: the latent carries the gradient, the diffusion model is constant
        _, _, hidden_v = self._denoise(latent, t, noise, frozen=True)
        if hidden_v.shape[:2] != targets.shape[:2]:
            raise ValueError(f"the model's {hidden_v.shape[1]} tokens at {self.alignment.layer!r} do not match the encoder's {targets.shape[1]} patches")
        vae_align = self._align(hidden_v, targets, frozen=True)
        # the diffusion model's terms on the detached latent
        out, target, hidden_d = self._denoise(latent.detach(), t, noise, frozen=False)
        err = 0.5 * (out - target.detach()) ** 2
        w = expand(self.process.weight(t).to(dev), err)
        denoise = (err * w).reshape(rows, -1).mean(1)
        dit_align = self._align(hidden_d, targets, frozen=False)
        per_row = vae_own + self.vae_align * vae_align + denoise + 0.5 * self.alignment.weight * dit_align
        mass = torch.tensor(float(rows), device=dev)
        metrics = {"denoising": Ratio(denoise.sum().detach(), mass), "reconstruction": Ratio(vae_own.sum().detach(), mass),
                   "alignment": Ratio(dit_align.sum().detach(), mass), "latent_alignment": Ratio(vae_align.sum().detach(), mass),
                   "latent_std": Ratio(latent.detach().std() * mass, mass)}
        return Ratio(per_row.sum(), mass), Aux(metrics=metrics)

    def generate(self, variables, shape, **kw):
        """Sample latents with the diffusion model and decode them with the jointly trained autoencoder."""
        self.autoencoder = None
        z = super().generate(variables, shape, **kw)
        return self.vae.decode(z)
