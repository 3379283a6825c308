"""DiLoCo: replicas train independently for ``every`` inner steps, then average their parameter *change* across the
``diloco`` axis and apply it with an outer optimizer (Nesterov momentum SGD on the pseudo-gradient).

Parity: src/dew/training/diloco.py:1-334 (outer axis, ``pmean`` every N updates, outer optimizer), src/dew/state.py
``TrainState.inner``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Optional

import torch
import torch.distributed as dist


@dataclass
class DiLoCoConfig:
    every: int = 100
    outer_lr: float = 0.7
    momentum: float = 0.9
    nesterov: bool = True


class DiLoCo:
    def __init__(self, params: Iterable[torch.nn.Parameter], config: DiLoCoConfig = DiLoCoConfig(), group: Optional[dist.ProcessGroup] = None):
        self.params = [p for p in params]
        self.cfg, self.group = config, group
        self.anchor = [p.detach().float().clone() for p in self.params]       # the last agreed (outer) weights
        self.velocity = [torch.zeros_like(a) for a in self.anchor]
        self.inner_steps = 0

    def after_inner_step(self) -> bool:
        """Call after every optimizer step; returns True when an outer step was taken."""
        self.inner_steps += 1
        if self.inner_steps % self.cfg.every:
            return False
        self.outer_step()
        return True

    @torch.no_grad()
    def outer_step(self) -> None:
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        for p, a, v in zip(self.params, self.anchor, self.velocity):
            delta = a - p.detach().float()                                     # pseudo-gradient: how far this replica moved
            if world > 1:
                dist.all_reduce(delta, group=self.group)
                delta /= world
            v.mul_(self.cfg.momentum).add_(delta)
            step = delta + self.cfg.momentum * v if self.cfg.nesterov else v
            a.sub_(self.cfg.outer_lr * step)
            p.copy_(a.to(p.dtype))
