"""``DiffusionObjective``: denoising loss for any ``Process`` (EDM, flow matching, VP ...), with classifier-free
condition dropout, EMA, and sampling-based ``evaluate`` / ``preview``.

Parity: src/dew/objectives/diffusion/objective.py (``__init__`` :432-548, ``loss`` :842-900, ``_denoised`` :902-930,
``_sample_impl`` :964-974).  Loss = half squared error x weight(t), row-mean, pooled as ``Ratio(total, mass)``.
"""
from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from ..diffusion import EDM, Process
from ..diffusion.schedules import expand
from ..inputs import Field, InputSpec
from ..sampling import CFG, DDIM, sample
from ..utils import keys as K
from .base import Aux, Objective, Ratio, Step


class DiffusionObjective(Objective):
    def __init__(self, model, process: Optional[Process] = None, inputs: Optional[InputSpec] = None, *,
                 autoencoder=None, unconditional_prob: float = 0.12, ema_decay: Optional[float] = 0.999,
                 solver=None, guidance=CFG(3.0), steps: Optional[int] = None, variables=None, uncertainty=None,
                 sample_shape=None):
        self.model = model
        if process is None:
            process = EDM(regime="latent" if autoencoder is not None else "pixel")()
        elif not isinstance(process, Process):
            process = process()  # a preset
        self.process = process
        self.inputs = inputs or InputSpec(Field("sample", tuple(sample_shape) if sample_shape else ()))
        self.autoencoder = autoencoder
        self.unconditional_prob = unconditional_prob
        self.ema_decay = ema_decay
        self.solver = solver if solver is not None else DDIM()
        self.guidance = guidance
        self.steps = steps or 200
        self.uncertainty = uncertainty
        self._given = variables

    def init(self, key=0, variables=None):
        return super().init(key, variables if variables is not None else self._given)

    def _conditions(self, batch, step: Step, rows: int, drop: bool):
        out = {}
        for name, cond in self.inputs.conditions.items():
            if cond.field.key not in batch:
                continue
            v = batch[cond.field.key]
            if cond.encoder is not None:
                v = cond.encoder(v)
            p = self.unconditional_prob if cond.dropout is None else cond.dropout
            if drop and p > 0:
                u = step.sample(f"drop/{name}", (), rows, kind="uniform").to(v.device)
                null = torch.zeros_like(v) if cond.null is None else torch.as_tensor(cond.null).to(v).expand_as(v)
                v = torch.where((u < p).reshape(-1, *([1] * (v.dim() - 1))), null, v)
            out[name] = v
        return out

    def loss(self, variables, batch: Mapping[str, torch.Tensor], step: Step):
        x0 = batch[self.inputs.sample.key]
        if self.autoencoder is not None:
            with torch.no_grad():
                x0 = self.autoencoder.encode(x0)
        x0 = x0.float()
        rows = x0.shape[0]
        dev = x0.device
        sched, pred = self.process.schedule, self.process.prediction
        # per-example draws: training time and noise
        tkeys = step.row_keys("time", rows)
        t = torch.stack([sched.sample_t(k, 1)[0] for k in tkeys]).to(dev)
        noise = step.sample("noise", x0.shape[1:], rows).to(dev)
        rates = self.process.rates(t, like=x0)
        x_t, c_in, target = pred.forward_diffusion(x0, noise, rates)
        conditions = self._conditions(batch, step, rows, drop=step.train)
        raw = self.apply(variables, x_t * c_in, sched.model_time(t), conditions, train=step.train).float()
        out = pred.pred_transform(x_t, raw, rates, t)
        err = 0.5 * (out - target) ** 2                       # optax.l2_loss: half squared error
        w = expand(self.process.weight(t).to(dev), err)
        per_row = (err * w).reshape(rows, -1).mean(1)
        mask = batch.get(self.inputs.mask.key) if self.inputs.mask is not None else None
        if mask is not None:
            m = mask.float().reshape(rows)
            stat = Ratio((per_row * m).sum(), m.sum())
        else:
            stat = Ratio(per_row.sum(), torch.tensor(float(rows), device=dev))
        return stat, Aux(metrics={"sigma_mean": Ratio(rates[1].reshape(rows, -1)[:, 0].sum(), torch.tensor(float(rows), device=dev))})

    def denoiser(self, variables, conditions=None):
        return self.process.denoiser(self.model, variables, conditions or {})

    def generate(self, variables, shape, *, key=0, conditions=None, steps=None, solver=None, guidance="default"):
        """Sample ``shape`` (including the batch axis) from the prior with the objective's solver and guidance."""
        den = self.denoiser(variables, conditions)
        dev = next(self.model.parameters()).device
        x_T = self.process.noise(K.fold_in(K.key(key), "prior"), shape).to(dev)
        g = self.guidance if guidance == "default" else guidance
        if not conditions:
            g = None
        x = sample(den, x_T, steps or self.steps, solver=solver or self.solver, guidance=g, key=key)
        if self.autoencoder is not None:
            x = self.autoencoder.decode(x)
        return x

    def preview(self, variables, batch=None, key=0, rows: int = 4, steps: Optional[int] = None, **kw):
        shape = self.inputs.sample.shape
        if batch is not None:
            shape = tuple(batch[self.inputs.sample.key].shape[1:])
        conditions = None
        if batch is not None and self.inputs.conditions:
            conditions = self._conditions({k: v[:rows] for k, v in batch.items()}, Step(), rows, drop=False)
        from ..utils.artifacts import ImageGrid
        imgs = self.generate(variables, (rows, *shape), key=key, conditions=conditions, steps=steps or min(self.steps, 20))
        return ImageGrid(imgs.clamp(-1, 1))

    def model_flops(self, batch):
        x = batch[self.inputs.sample.key]
        fn = getattr(self.model, "model_flops", None)
        if fn is None:
            return None
        p = getattr(self.model, "patch_size", 1)
        return fn((x.shape[1] // p) * (x.shape[2] // p), x.shape[0])
