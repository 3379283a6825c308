"""``Objective``: what a run optimises.  ``loss(variables, batch, step)`` returns exactly poolable statistics
(``Ratio(total, mass)`` etc.), optionally with an ``Aux`` of metrics and non-parameter effects.

Parity: src/dew/objectives/base.py (statistics :129-270, ``Step`` :411-581, ``Aux`` :600-655, ``EMASpec`` :768,
``Objective`` :902-2056).  Statistics are sums and masses that add exactly across microbatches and ranks and are
divided once; per-example draws are keyed by the example's global index so they do not depend on batch layout.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Any, Callable, Dict, Mapping, Optional, Sequence, Tuple

import torch

from ..utils import keys as K
from ..utils.trees import module_variables, variables_for_call


# ------------------------------------------------------------------------------------------------ statistics
@dataclass
class Ratio:
    """``total / mass`` pooled exactly: both are sums."""
    total: torch.Tensor
    mass: torch.Tensor

    def __add__(self, other: "Ratio") -> "Ratio":
        return Ratio(self.total + other.total, self.mass + other.mass)

    def value(self) -> torch.Tensor:
        return self.total / torch.as_tensor(self.mass, dtype=self.total.dtype, device=self.total.device).clamp_min(1e-12)

    def parts(self):
        return [self.total, torch.as_tensor(self.mass, dtype=torch.float32, device=self.total.device)]

    @classmethod
    def of(cls, parts):
        return cls(parts[0], parts[1])


def Mean(values: torch.Tensor, weights: Optional[torch.Tensor] = None) -> Ratio:
    v = values.float()
    if weights is None:
        return Ratio(v.sum(), torch.tensor(float(v.numel()), device=v.device))
    w = weights.float()
    return Ratio((v * w).sum(), w.sum())


@dataclass
class Summed:
    total: torch.Tensor

    def __add__(self, o):
        return Summed(self.total + o.total)

    def value(self):
        return self.total

    def parts(self):
        return [self.total]

    @classmethod
    def of(cls, parts):
        return cls(parts[0])


@dataclass
class Moments:
    """Count, sum and sum of squares -> mean and variance."""
    count: torch.Tensor
    s1: torch.Tensor
    s2: torch.Tensor

    @classmethod
    def from_values(cls, v: torch.Tensor) -> "Moments":
        v = v.float()
        return cls(torch.tensor(float(v.numel()), device=v.device), v.sum(), (v * v).sum())

    def __add__(self, o):
        return Moments(self.count + o.count, self.s1 + o.s1, self.s2 + o.s2)

    def mean(self):
        return self.s1 / self.count.clamp_min(1)

    def variance(self):
        m = self.mean()
        return (self.s2 / self.count.clamp_min(1) - m * m).clamp_min(0)

    def value(self):
        return self.mean()

    def parts(self):
        return [self.count, self.s1, self.s2]

    @classmethod
    def of(cls, parts):
        return cls(*parts)


@dataclass
class Exponentiated:
    """exp of a pooled ratio (perplexity from summed negative log-likelihood)."""
    inner: Ratio

    def __add__(self, o):
        return Exponentiated(self.inner + o.inner)

    def value(self):
        return torch.exp(self.inner.value())

    def parts(self):
        return self.inner.parts()

    @classmethod
    def of(cls, parts):
        return cls(Ratio.of(parts))


@dataclass
class Weighted:
    """A statistic scaled by a fixed coefficient when read."""
    inner: Any
    weight: float = 1.0

    def __add__(self, o):
        return Weighted(self.inner + o.inner, self.weight)

    def value(self):
        return self.inner.value() * self.weight

    def parts(self):
        return self.inner.parts()


Pooled = (Ratio, Summed, Moments, Exponentiated, Weighted)


def pool(stats: Sequence[Any]) -> Any:
    out = stats[0]
    for s in stats[1:]:
        out = out + s
    return out


# ------------------------------------------------------------------------------------------------ step / aux / ema
@dataclass
class Step:
    """Per-step context handed to ``loss``: the step index, the step's key and the EMA variables if kept.

    ``sample(name, shape, indices=...)`` draws one independent row per example, keyed by the example's global
    index, so a row's noise is the same on any rank / microbatch split.
    """
    step: int = 0
    key: K.Key = 0
    ema: Optional[Mapping[str, Any]] = None
    train: bool = True
    first_index: int = 0        # global index of this (micro)batch's first example within the step
    device: Any = "cpu"

    def fold(self, name: str) -> K.Key:
        return K.fold_in(self.key, name)

    def sample(self, name: str, shape: Sequence[int], rows: int, kind: str = "normal", **kw) -> torch.Tensor:
        base = self.fold(name)
        draw = {"normal": K.normal, "uniform": K.uniform}[kind]
        out = K.per_example(base, range(self.first_index, self.first_index + rows), draw, shape, **kw)
        return out.to(self.device)

    def row_keys(self, name: str, rows: int):
        base = self.fold(name)
        return [K.fold_in(base, i) for i in range(self.first_index, self.first_index + rows)]


@dataclass
class Aux:
    """The one channel for everything a loss returns besides its statistic: metrics (poolable statistics) and
    effects (non-parameter updates such as a router's balancing bias or batch statistics)."""
    metrics: Dict[str, Any] = field(default_factory=dict)
    effects: Dict[str, Any] = field(default_factory=dict)
    sown: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class EMASpec:
    """How the weight average decays: a constant, a warm-up ``min(decay, (1+n)/(10+n))`` or a power profile
    (``decay_n = (1 - 1/n)^(gamma+1)``, Karras et al. 2024)."""
    decay: float = 0.999
    kind: str = "constant"
    gamma: float = 0.0
    start: int = 0

    @classmethod
    def constant(cls, decay: float) -> "EMASpec":
        return cls(decay=decay, kind="constant")

    @classmethod
    def warmup(cls, decay: float) -> "EMASpec":
        return cls(decay=decay, kind="warmup")

    @classmethod
    def power(cls, std: float) -> "EMASpec":
        from ..optim.averaging import gamma_of_std
        return cls(kind="power", gamma=gamma_of_std(std))

    def at(self, updates: int) -> float:
        if updates < self.start:
            return 0.0
        if self.kind == "constant":
            return self.decay
        if self.kind == "warmup":
            return min(self.decay, (1 + updates) / (10 + updates))
        if self.kind == "power":
            n = max(updates, 1)
            return (1 - 1 / n) ** (self.gamma + 1)
        raise ValueError(f"unknown EMA kind {self.kind!r}")


# ------------------------------------------------------------------------------------------------ objective
class Objective:
    """Base class.  Subclasses set ``self.model`` (an ``nn.Module``) and implement ``loss``."""
    model: torch.nn.Module
    ema_decay: Optional[float] = None
    starts_from_model: bool = False     # fine-tuning objectives (preference / policy optimisation): ``init`` keeps the module's
                                        # current weights instead of drawing new ones when no starting tree is given

    # -- construction of state
    def init(self, key: K.Key = 0, variables: Optional[Mapping[str, Any]] = None) -> Dict[str, Any]:
        """Initialise (or adopt) the variables: a ``{'params': tree}`` whose leaves alias the model's parameters."""
        from ..nn.layers import reset_all
        if variables is None:
            if not self.starts_from_model:
                reset_all(self.model, int(key) & 0x7FFFFFFF)
            return module_variables(self.model)
        flat = variables_for_call(self.model, variables)
        with torch.no_grad():
            for name, p in self.model.named_parameters():
                if name in flat:
                    p.copy_(flat[name])
        return module_variables(self.model)

    def ema_spec(self) -> Optional[EMASpec]:
        d = self.ema_decay
        if d is None:
            return None
        return d if isinstance(d, EMASpec) else EMASpec.constant(float(d))

    # -- applying the model functionally
    def apply(self, variables: Optional[Mapping[str, Any]], *args, **kwargs):
        if variables is None:
            return self.model(*args, **kwargs)
        return torch.func.functional_call(self.model, variables_for_call(self.model, variables), args, kwargs)

    # -- the contract
    def loss(self, variables, batch, step: Step):
        raise NotImplementedError

    def reduce_loss(self, stats) -> Tuple[torch.Tensor, torch.Tensor]:
        """``(scalar loss to differentiate, mass)``; the trainer divides the pooled total by the pooled mass."""
        if isinstance(stats, Ratio):
            return stats.total, stats.mass
        if isinstance(stats, (Moments,)):
            return stats.s1, stats.count
        return stats.value(), torch.tensor(1.0)

    def evaluate(self, variables, batch, step: Step) -> Dict[str, Any]:
        with torch.no_grad():
            out = self.loss(variables, batch, replace(step, train=False))
        stats, aux = out if isinstance(out, tuple) else (out, Aux())
        return {"loss": stats, **aux.metrics}

    def preview(self, variables, batch=None, key: K.Key = 0, **kw):
        return None

    def predict(self, variables, batch):
        raise NotImplementedError

    def optimizer(self, tx):
        return tx

    def apply_effects(self, variables, effects: Mapping[str, Any]):
        """Write non-parameter updates (``Aux.effects``) back; default: buffers by path."""
        from ..utils.trees import flatten
        if not effects:
            return
        bufs = dict(self.model.named_buffers())
        with torch.no_grad():
            for name, value in effects.items():
                if name in bufs:
                    bufs[name].copy_(value)

    def model_flops(self, batch) -> Optional[float]:
        return None

    def training_flops(self, batch) -> Optional[float]:
        f = self.model_flops(batch)
        return None if f is None else 3.0 * f

    def scored_tokens(self, batch) -> Optional[int]:
        return None

    def row_tokens(self, batch) -> Optional[int]:
        return None

    def pipeline(self, state, ema: Optional[bool] = None):
        raise NotImplementedError(f"{type(self).__name__} declares no inference task")

    def placement(self, layout):
        return layout

    def data(self, tokenizer=None):
        return None

    # -- helpers
    @staticmethod
    def row_mean(values: torch.Tensor) -> torch.Tensor:
        return values.float().reshape(values.shape[0], -1).mean(1)

    @staticmethod
    def row_moments(values: torch.Tensor) -> Moments:
        return Moments.from_values(values)

    @staticmethod
    def accuracy(logits: torch.Tensor, targets: torch.Tensor, mask: Optional[torch.Tensor] = None) -> Ratio:
        hit = (logits.argmax(-1) == targets).float()
        return Mean(hit, mask)


@dataclass
class Metric:
    name: str
    fn: Callable[..., Any]
    every: Optional[int] = None
