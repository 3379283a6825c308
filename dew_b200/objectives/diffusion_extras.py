"""Two diffusion objectives built on ``DiffusionObjective``: representation alignment (REPA / iREPA) and guidance
distillation.

``AlignedDiffusionObjective`` adds to the denoising loss the negative cosine similarity between a frozen encoder's patch
features of the clean image and a projection of the denoiser's hidden tokens at one layer (Yu et al. 2025; iREPA: a
convolutional projector and spatially z-scored targets).  The hidden tokens are read with a forward hook on the named
submodule, the projector lives beside the backbone in one module so the trainer optimises both.

``GuidanceDistillationObjective`` trains a student that reads the guidance scale as an input to match a frozen teacher's
classifier-free guided raw output at a scale drawn per example (Meng et al. 2023, stage one).

Reference: src/dew/objectives/diffusion/alignment.py (``Projector`` :44, ``spatial_zscore`` :70, ``Alignment`` :83-193),
src/dew/objectives/diffusion/guidance_distillation.py (``GuidanceDistillationObjective`` :41-146).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..diffusion.schedules import expand
from .base import Aux, Ratio, Step
from .diffusion import DiffusionObjective

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


class Projector(nn.Module):
    """Hidden tokens ``[B, N, width_in]`` -> ``[B, N, features]``: REPA's MLP (two hidden SiLU layers of ``width``) or iREPA's
    single same-padded convolution over the (square) token grid."""

    def __init__(self, kind: str, in_features: int, features: int, width: int = 2048, kernel_size: int = 3):
        super().__init__()
        if kind not in ("mlp", "conv"):
            raise ValueError(f"projector is mlp or conv, not {kind!r}")
        self.kind = kind
        if kind == "mlp":
            self.net = nn.Sequential(nn.Linear(in_features, width), nn.SiLU(), nn.Linear(width, width), nn.SiLU(), nn.Linear(width, features))
        else:
            self.net = nn.Conv2d(in_features, features, kernel_size, padding=kernel_size // 2)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        if self.kind == "mlp":
            return self.net(tokens)
        B, N, W = tokens.shape
        side = math.isqrt(N)
        if side * side != N:
            raise ValueError(f"a convolution projector needs a square token grid, not {N} tokens")
        grid = self.net(tokens.reshape(B, side, side, W).permute(0, 3, 1, 2))
        return grid.permute(0, 2, 3, 1).reshape(B, N, -1)


def spatial_zscore(features: torch.Tensor, gamma: float) -> torch.Tensor:
    """iREPA's spatial normalisation of ``[B, N, D]``: subtract ``gamma`` x the mean over tokens, divide by the unbiased
    standard deviation over tokens plus 1e-6."""
    mean = features.mean(1, keepdim=True)
    std = features.std(1, keepdim=True, unbiased=True)
    return (features - gamma * mean) / (std + 1e-6)


@dataclass
class Alignment:
    """What to align: the output of submodule ``layer`` of the backbone (a ``[B, N, width]`` token sequence in raster order)
    with ``encoder(pixels) -> [B, N, D]`` or ``[B, h, w, D]`` patch features.  ``weight`` is REPA's ``proj_coeff``; the loss
    adds ``weight / 2`` x the alignment term because the denoising error here is the half squared error.  Pixels in
    ``[-1, 1]`` are mapped to ``[0, 1]``, normalised by ``mean`` / ``std`` and resized (bicubic) to ``resolution``."""
    layer: str = "blocks.7"
    encoder: Optional[Callable] = None
    weight: float = 0.5
    projector: str = "mlp"
    width: int = 2048
    kernel_size: int = 3
    spatial_norm: Optional[float] = None
    resolution: Optional[int] = 224
    mean: Tuple[float, float, float] = IMAGENET_MEAN
    std: Tuple[float, float, float] = IMAGENET_STD

    def __post_init__(self):
        if self.projector not in ("mlp", "conv"):
            raise ValueError(f"projector is mlp or conv, not {self.projector!r}")
        if self.encoder is None:
            raise ValueError("the alignment needs an encoder: a callable from pixels [B, H, W, 3] to patch features "
                             "(pretrained weights are loaded by the caller, e.g. through dew_b200.interop)")

    @torch.no_grad()
    def targets(self, images: torch.Tensor) -> torch.Tensor:
        px = (images.float() + 1) / 2
        px = (px - torch.tensor(self.mean, device=px.device)) / torch.tensor(self.std, device=px.device)
        if self.resolution is not None and self.resolution != px.shape[1]:
            px = F.interpolate(px.permute(0, 3, 1, 2), size=(self.resolution, self.resolution), mode="bicubic",
                               align_corners=False).permute(0, 2, 3, 1)
        f = self.encoder(px)
        if not isinstance(f, torch.Tensor):
            raise TypeError("a representation encoder must return one tensor of patch features")
        f = f.reshape(f.shape[0], -1, f.shape[-1]).float()
        return spatial_zscore(f, self.spatial_norm) if self.spatial_norm is not None else f


class AlignedModel(nn.Module):
    """Backbone + alignment projector in one module (the trainer optimises ``objective.model``).  Calls go to the backbone;
    a forward hook on ``layer`` keeps that call's hidden tokens in ``self.hidden``."""

    def __init__(self, backbone: nn.Module, projector: Projector, layer: str):
        super().__init__()
        self.backbone, self.alignment_projector = backbone, projector
        self.hidden: Optional[torch.Tensor] = None
        backbone.get_submodule(layer).register_forward_hook(self._keep)

    def _keep(self, module, args, output):
        self.hidden = output[0] if isinstance(output, tuple) else output

    def forward(self, *args, **kwargs):
        return self.backbone(*args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("backbone"), name)


class AlignedDiffusionObjective(DiffusionObjective):
    """``DiffusionObjective`` + ``alignment.weight / 2 * mean(-cos(projector(hidden), encoder(clean image)))``.  The hidden
    width is probed once from the backbone (``hidden_features`` or the first call); ``encoder_features`` is the encoder's D."""

    def __init__(self, model: nn.Module, process=None, inputs=None, *, alignment: Alignment, hidden_features: int,
                 encoder_features: int, **kw):
        self.alignment = alignment
        proj = Projector(alignment.projector, hidden_features, encoder_features, alignment.width, alignment.kernel_size)
        p = next(model.parameters(), None)
        if p is not None:
            proj = proj.to(p.device)
        super().__init__(AlignedModel(model, proj, alignment.layer), process, inputs, **kw)

    def loss(self, variables, batch, step: Step):
        stat, aux = super().loss(variables, batch, step)
        hidden = self.model.hidden
        if hidden is None:
            raise RuntimeError(f"the backbone's submodule {self.alignment.layer!r} did not run in this call")
        images = batch[self.inputs.sample.key]
        targets = self.alignment.targets(images)
        if hidden.shape[:2] != targets.shape[:2]:
            raise ValueError(f"the model's {hidden.shape[1]} tokens at {self.alignment.layer!r} do not match the encoder's "
                             f"{targets.shape[1]} patches")
        from ..utils.trees import variables_for_call
        flat = variables_for_call(self.model, variables) if variables is not None else None
        if flat is not None:
            sub = {k[len("alignment_projector."):]: v for k, v in flat.items() if k.startswith("alignment_projector.")}
            projected = torch.func.functional_call(self.model.alignment_projector, sub, (hidden.float(),))
        else:
            projected = self.model.alignment_projector(hidden.float())
        cos = F.cosine_similarity(projected.float(), targets, dim=-1).mean(1)            # [B]
        rows = cos.shape[0]
        mask = batch.get(self.inputs.mask.key) if self.inputs.mask is not None else None
        m = mask.float().reshape(rows) if mask is not None else torch.ones(rows, device=cos.device)
        align = Ratio(-(cos * m).sum(), m.sum())
        aux.metrics["alignment"] = Ratio(align.total.detach(), align.mass)
        self.model.hidden = None
        return Ratio(stat.total + 0.5 * self.alignment.weight * align.total, stat.mass), aux


def guide(conditional: torch.Tensor, unconditional: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Classifier-free guidance with one scale per row: ``uncond + w (cond - uncond)``."""
    return unconditional + expand(scale.to(conditional.device), conditional) * (conditional - unconditional)


class GuidanceDistillationObjective(DiffusionObjective):
    """The student reads ``conditions["guidance"]`` (one scale per row, uniform in ``scales``) and regresses its raw output
    onto the frozen teacher's guided raw output at that scale, on the same noised sample, under the process's weighting.
    The teacher is a module over the same process and inputs (default: a frozen copy of the student at construction); its
    unconditional branch reads each condition's null value.  Sampling from the student is unguided."""

    def __init__(self, model: nn.Module, process=None, inputs=None, *, teacher: Optional[nn.Module] = None,
                 scales: Tuple[float, float] = (1.0, 8.0), **kw):
        kw.setdefault("guidance", None)
        super().__init__(model, process, inputs, **kw)
        if teacher is None:
            import copy
            teacher = copy.deepcopy(model)
        self.teacher = teacher.requires_grad_(False).eval()
        low, high = scales
        if not (low <= high):
            raise ValueError("scales is (low, high) with low <= high")
        self.scales = (float(low), float(high))
        if not self.inputs.conditions:
            raise ValueError("guidance distillation needs a conditioned model: there is nothing to guide without conditions")

    def _null(self, conditions: Mapping[str, torch.Tensor]) -> dict:
        out = {}
        for name, v in conditions.items():
            cond = self.inputs.conditions[name]
            out[name] = torch.zeros_like(v) if cond.null is None else torch.as_tensor(cond.null).to(v).expand_as(v)
        return out

    def loss(self, variables, batch, step: Step):
        x0 = batch[self.inputs.sample.key]
        if self.autoencoder is not None:
            with torch.no_grad():
                x0 = self.autoencoder.encode(x0)
        x0 = x0.float()
        rows, dev = x0.shape[0], x0.device
        sched, pred = self.process.schedule, self.process.prediction
        low, high = self.scales
        scale = (low + (high - low) * step.sample("guidance scale", (), rows, kind="uniform")).to(dev)
        t = torch.stack([sched.sample_t(k, 1)[0] for k in step.row_keys("time", rows)]).to(dev)
        noise = step.sample("noise", x0.shape[1:], rows).to(dev)
        rates = self.process.rates(t, like=x0)
        x_t, c_in, _ = pred.forward_diffusion(x0, noise, rates)
        given = self._conditions(batch, step, rows, drop=False)
        time = sched.model_time(t)
        with torch.no_grad():
            cond = self.teacher(x_t * c_in, time, given).float()
            uncond = self.teacher(x_t * c_in, time, self._null(given)).float()
            target = guide(cond, uncond, scale)
        out = self.apply(variables, x_t * c_in, time, {**given, "guidance": scale}, train=step.train).float()
        err = 0.5 * (out - target) ** 2
        w = expand(self.process.weight(t).to(dev), err)
        per_row = (err * w).reshape(rows, -1).mean(1)
        return Ratio(per_row.sum(), torch.tensor(float(rows), device=dev)), Aux(metrics={"guidance_scale": Ratio(scale.sum(), torch.tensor(float(rows), device=dev))})
