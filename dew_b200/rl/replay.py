"""A fixed-size ring replay buffer of named tensors with seeded uniform sampling.  Reference: src/dew/rl/replay.py."""
from __future__ import annotations

from typing import Dict, Mapping

import torch


class Replay:
    def __init__(self, capacity: int, device="cpu"):
        self.capacity, self.device = capacity, device
        self.store: Dict[str, torch.Tensor] = {}
        self.size = self.cursor = 0

    def add(self, batch: Mapping[str, torch.Tensor]) -> None:
        n = next(iter(batch.values())).shape[0]
        for k, v in batch.items():
            if k not in self.store:
                self.store[k] = torch.zeros((self.capacity,) + tuple(v.shape[1:]), dtype=v.dtype, device=self.device)
        idx = (self.cursor + torch.arange(n)) % self.capacity
        for k, v in batch.items():
            self.store[k][idx] = v.to(self.device)
        self.cursor = int((self.cursor + n) % self.capacity)
        self.size = min(self.capacity, self.size + n)

    def sample(self, n: int, generator: torch.Generator | None = None) -> Dict[str, torch.Tensor]:
        idx = torch.randint(0, self.size, (n,), generator=generator)
        return {k: v[idx] for k, v in self.store.items()}
