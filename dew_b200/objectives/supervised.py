"""``Supervised``: classification / regression on ``(inputs, targets)`` batches with a pluggable loss."""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .base import Aux, Mean, Objective, Ratio, Step


class Supervised(Objective):
    def __init__(self, model, loss: str = "cross_entropy", inputs_key: str = "inputs", targets_key: str = "targets",
                 ema_decay: Optional[float] = None, label_smoothing: float = 0.0):
        self.model, self.loss_kind, self.inputs_key, self.targets_key = model, loss, inputs_key, targets_key
        self.ema_decay, self.label_smoothing = ema_decay, label_smoothing

    def loss(self, variables, batch, step: Step):
        x, y = batch[self.inputs_key], batch[self.targets_key]
        out = self.apply(variables, x)
        rows = x.shape[0]
        if self.loss_kind == "cross_entropy":
            per = F.cross_entropy(out.float(), y, reduction="none", label_smoothing=self.label_smoothing)
            aux = Aux(metrics={"accuracy": self.accuracy(out, y)})
        elif self.loss_kind == "mse":
            per = ((out.float() - y.float()) ** 2).reshape(rows, -1).mean(1)
            aux = Aux()
        else:
            raise ValueError(f"unknown loss {self.loss_kind!r}; known: cross_entropy, mse")
        return Ratio(per.sum(), torch.tensor(float(rows), device=per.device)), aux

    def predict(self, variables, batch):
        return self.apply(variables, batch[self.inputs_key])
