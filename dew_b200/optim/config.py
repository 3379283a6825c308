"""``OptimConfig`` and the optimizers it builds.

Fields follow src/dew/optim.py:1863- (``optimizer="adamw"``, ``optimizer_opts``, ``learning_rate`` float | schedule,
``weight_decay`` (1e-4 default), ``spared`` (names that take no decay), ``param_groups``, ``clip_grads``,
``state_dtype``, ``ema_profiles``).  Optimizers: adamw (fused flat kernel), sgd, lamb, laprop, lion, muon
(Newton-Schulz orthogonalised momentum for 2-D weights, AdamW for the rest).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple, Union

import torch

from .. import ops
from ..utils.trees import flatten, unflatten
from .schedules import as_schedule


@dataclass
class OptimConfig:
    optimizer: str = "adamw"
    optimizer_opts: Dict[str, Any] = field(default_factory=dict)
    learning_rate: Union[float, Callable[[int], float]] = 1e-3
    weight_decay: float = 1e-4
    spared: Sequence[str] = ("bias", "scale", "norm", "embedding", "sinks", "A_log", "dt_bias")
    param_groups: Sequence[Mapping[str, Any]] = ()      # [{"match": regex, "learning_rate": x | "lr_scale": s, "weight_decay": w}]
    clip_grads: Optional[float] = None
    state_dtype: str = "float32"                         # float32 | bfloat16
    ema_profiles: Sequence[float] = ()                   # relative stds of post-hoc power profiles
    skip_nonfinite: bool = False

    def build(self) -> "Optimizer":
        return Optimizer(self)


def newton_schulz(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz iteration towards the orthogonal polar factor (Muon; src/dew/newton_schulz.py)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.float()
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.t()
    X = X / (X.norm() + 1e-7)
    for _ in range(steps):
        A = X @ X.t()
        X = a * X + (b * A + c * A @ A) @ X
    return X.t() if transposed else X


class Optimizer:
    """Functional-style optimizer over a flat ``path -> tensor`` view of the variables.

    ``init(params)`` creates the state; ``update(params, grads, state, step)`` updates params **in place** (masters)
    and returns the new state.  Leaves of ``state`` keep the parameter paths, so checkpoints name them
    ``opt_state/mu/<path>``.
    """

    def __init__(self, config: OptimConfig):
        self.config = config
        self.schedule = as_schedule(config.learning_rate)

    # ------------------------------------------------------------------ groups
    def _group_of(self, path: str) -> Tuple[float, float]:
        """(lr scale, weight decay) for a leaf."""
        cfg = self.config
        scale, wd = 1.0, cfg.weight_decay
        leaf = path.rsplit("/", 1)[-1]
        if any(s in leaf or s in path.split("/")[-2:-1] for s in cfg.spared) or leaf in ("bias",):
            wd = 0.0
        for g in cfg.param_groups:
            if re.search(g["match"], path):
                scale = g.get("lr_scale", scale)
                wd = g.get("weight_decay", wd)
        return scale, wd

    # ------------------------------------------------------------------ state
    def init(self, params: Mapping[str, Any]) -> Dict[str, Any]:
        flat = flatten(params)
        sd = torch.float32 if self.config.state_dtype == "float32" else torch.bfloat16
        zeros = lambda p: torch.zeros_like(p, dtype=sd if p.dtype.is_floating_point else p.dtype)
        state: Dict[str, Any] = {"count": torch.zeros((), dtype=torch.int64)}
        kind = self.config.optimizer
        if kind in ("adamw", "adam", "lamb", "laprop", "muon", "normuon"):
            state["mu"] = unflatten({k: zeros(v) for k, v in flat.items()})
            state["nu"] = unflatten({k: zeros(v) for k, v in flat.items()})
        elif kind == "m3":
            # fast momentum, second moment, slow momentum, the open chunk's gradient sum and the slow direction read by the
            # next chunk (fp32 at least: the sums do not decay)
            f32 = lambda p: torch.zeros_like(p, dtype=torch.float32 if p.dtype.is_floating_point else p.dtype)
            for name in ("mu", "nu", "slow", "chunk", "slow_direction"):
                state[name] = unflatten({k: f32(v) for k, v in flat.items()})
        elif kind in ("sgd", "lion"):
            state["mu"] = unflatten({k: zeros(v) for k, v in flat.items()})
        else:
            raise ValueError(f"unknown optimizer {kind!r}; known: adamw, adam, sgd, lamb, laprop, lion, muon, normuon, m3")
        return state

    # ------------------------------------------------------------------ gradient norm / clipping
    @staticmethod
    def global_norm(grads: Mapping[str, Any]) -> torch.Tensor:
        leaves = [g for g in flatten(grads).values() if g is not None]
        if not leaves:
            return torch.zeros(())
        return torch.sqrt(sum(g.float().pow(2).sum() for g in leaves))

    # ------------------------------------------------------------------ update
    @torch.no_grad()
    def update(self, params, grads, state, step: int, grad_scale: float = 1.0) -> Tuple[Dict[str, Any], Dict[str, Any]]:
        cfg = self.config
        opts = cfg.optimizer_opts
        p_flat, g_flat = flatten(params), flatten(grads)
        lr = float(self.schedule(step))
        count = int(state["count"]) + 1
        norm = self.global_norm(grads) * grad_scale
        info = {"grad_norm": norm, "learning_rate": lr}
        if cfg.skip_nonfinite and not bool(torch.isfinite(norm)):
            info["skipped"] = True
            return state, info
        coef = grad_scale
        if cfg.clip_grads is not None and float(norm) > cfg.clip_grads:
            coef = coef * cfg.clip_grads / (float(norm) + 1e-6)
        b1, b2, eps = opts.get("b1", 0.9), opts.get("b2", 0.999), opts.get("eps", 1e-8)
        mu, nu = flatten(state.get("mu", {})), flatten(state.get("nu", {}))
        kind = cfg.optimizer
        for path, p in p_flat.items():
            g = g_flat.get(path)
            if g is None or not p.dtype.is_floating_point:
                continue
            scale, wd = self._group_of(path)
            plr = lr * scale
            if kind in ("adamw", "adam"):
                wdk = wd if kind == "adamw" else 0.0
                if p.dtype == torch.float32 and mu[path].dtype == torch.float32 and p.is_contiguous():
                    ops.adamw_(p.view(-1), mu[path].view(-1), nu[path].view(-1), g.reshape(-1), step=count, lr=plr,
                               beta1=b1, beta2=b2, eps=eps, weight_decay=wdk, grad_scale=coef)
                else:
                    _adamw_generic(p, mu[path], nu[path], g, count, plr, b1, b2, eps, wdk, coef)
            elif kind == "sgd":
                m = mu[path]
                m.mul_(opts.get("momentum", 0.9)).add_(g.to(m.dtype), alpha=coef)
                p.mul_(1 - plr * wd).add_(m.to(p.dtype), alpha=-plr)
            elif kind == "lion":
                m = mu[path]
                gf = g.float() * coef
                upd = torch.sign(m.float() * b1 + gf * (1 - b1))
                p.mul_(1 - plr * wd).add_(upd.to(p.dtype), alpha=-plr)
                m.copy_((m.float() * b2 + gf * (1 - b2)).to(m.dtype))
            elif kind == "laprop":
                gf = g.float() * coef
                nu[path].copy_((nu[path].float() * b2 + (1 - b2) * gf * gf).to(nu[path].dtype))
                den = (nu[path].float() / (1 - b2 ** count)).sqrt() + eps
                mu[path].copy_((mu[path].float() * b1 + (1 - b1) * gf / den).to(mu[path].dtype))
                p.mul_(1 - plr * wd).add_((mu[path].float() / (1 - b1 ** count)).to(p.dtype), alpha=-plr)
            elif kind == "lamb":
                gf = g.float() * coef
                mu[path].copy_((mu[path].float() * b1 + (1 - b1) * gf).to(mu[path].dtype))
                nu[path].copy_((nu[path].float() * b2 + (1 - b2) * gf * gf).to(nu[path].dtype))
                upd = (mu[path].float() / (1 - b1 ** count)) / ((nu[path].float() / (1 - b2 ** count)).sqrt() + eps) + wd * p.float()
                wn, un = p.float().norm(), upd.norm()
                trust = float(wn / un) if float(wn) > 0 and float(un) > 0 else 1.0
                p.add_(upd.to(p.dtype), alpha=-plr * trust)
            elif kind == "m3":
                # Multi-scale Momentum Muon (Nested Learning, arXiv 2512.24695, Algorithm 1): direction
                # (O1 + alpha O2) / sqrt(V + eps); M1 += beta1 g, V += beta2 g^2 (sums, no decay); every `frequency` updates
                # the slow momentum M2 += beta3 * (the chunk's gradient sum) and O2 = orthogonalised M2 for the next chunk.
                slow, chunk, sdir = (flatten(state[n]) for n in ("slow", "chunk", "slow_direction"))
                gf = g.float() * coef
                beta3, alpha, freq = opts.get("b3", 0.9), opts.get("alpha", 0.5), int(opts.get("frequency", 4))
                mu[path].add_(gf, alpha=opts.get("b1", 0.9))
                nu[path].add_(gf * gf, alpha=opts.get("b2", 0.999))
                matrix = p.dim() == 2
                o1 = newton_schulz(mu[path], opts.get("ns_steps", 5)) if matrix else mu[path] / (mu[path].norm() + 1e-7)
                direction = (o1 + alpha * sdir[path]) / torch.sqrt(nu[path] + opts.get("eps", 1e-8))
                p.mul_(1 - plr * wd).add_(direction.to(p.dtype), alpha=-plr)
                chunk[path].add_(gf)
                if count % freq == 0:
                    slow[path].add_(chunk[path], alpha=beta3)
                    chunk[path].zero_()
                    sdir[path].copy_(newton_schulz(slow[path], opts.get("ns_steps", 5)) if matrix else slow[path] / (slow[path].norm() + 1e-7))
            elif kind == "normuon":
                # NorMuon (arXiv 2510.05491): Muon's orthogonal update, each output neuron (row) divided by the root of its
                # decayed mean square, the matrix scaled back to the orthogonal update's Frobenius norm
                if p.dim() == 2 and "embed" not in path and "head" not in path:
                    m = mu[path]
                    mom = opts.get("momentum", 0.95)
                    m.mul_(mom).add_(g.to(m.dtype), alpha=coef)
                    u = newton_schulz(g.float() * coef + mom * m.float(), opts.get("ns_steps", 5))
                    row = nu[path][:, :1]
                    b2n = opts.get("neuron_b2", 0.95)
                    row.copy_((row.float() * b2n + (1 - b2n) * u.pow(2).mean(1, keepdim=True)).to(row.dtype))
                    normed = u / (row.float().sqrt() + opts.get("neuron_eps", 1e-10))
                    normed = normed * (u.norm() / (normed.norm() + 1e-20))
                    normed = normed * max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                    p.mul_(1 - plr * wd).add_(normed.to(p.dtype), alpha=-plr)
                else:
                    _adamw_generic(p, mu[path], nu[path], g, count, plr * opts.get("adam_lr_scale", 1.0), b1, b2, eps, wd, coef)
            elif kind == "muon":
                if p.dim() == 2 and "embed" not in path and "head" not in path:
                    m = mu[path]
                    m.mul_(opts.get("momentum", 0.95)).add_(g.to(m.dtype), alpha=coef)
                    u = newton_schulz(g.float() * coef + opts.get("momentum", 0.95) * m.float(), opts.get("ns_steps", 5))
                    u = u * max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                    p.mul_(1 - plr * wd).add_(u.to(p.dtype), alpha=-plr)
                else:
                    _adamw_generic(p, mu[path], nu[path], g, count, plr * opts.get("adam_lr_scale", 1.0), b1, b2, eps, wd, coef)
        new_state = dict(state)
        new_state["count"] = torch.tensor(count, dtype=torch.int64)
        return new_state, info


def _adamw_generic(p, m, v, g, count, lr, b1, b2, eps, wd, coef):
    gf = g.float() * coef
    mf = m.float() * b1 + (1 - b1) * gf
    vf = v.float() * b2 + (1 - b2) * gf * gf
    m.copy_(mf.to(m.dtype))
    v.copy_(vf.to(v.dtype))
    upd = (mf / (1 - b1 ** count)) / ((vf / (1 - b2 ** count)).sqrt() + eps)
    p.copy_((p.float() * (1 - lr * wd) - lr * upd).to(p.dtype))
