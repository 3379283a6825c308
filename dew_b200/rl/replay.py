"""Replays of environment steps held on the device.

``ReplayBuffer`` keeps the last ``capacity`` steps of each of ``envs`` environments - a ring per environment over a tree of step
fields ``[capacity, envs, ...]`` - and ``sample`` draws uniformly among the windows of ``length`` consecutive steps it holds whole
(DreamerV3's uniform replay of chunks).  ``Replay`` is the flat ring of independent rows with seeded uniform sampling.

Reference: src/dew/rl/replay.py (``ReplayBuffer``: ``held``, ``cursor``, ``filled``, ``add``, ``sample``).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

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

    def sample(self, n: int, generator: Optional[torch.Generator] = None) -> Dict[str, torch.Tensor]:
        idx = torch.randint(0, self.size, (n,), generator=generator)
        return {k: v[idx] for k, v in self.store.items()}


class ReplayBuffer:
    def __init__(self, capacity: int, envs: int, device="cpu"):
        self.capacity, self.envs, self.device = capacity, envs, torch.device(device)
        self.held: Dict[str, torch.Tensor] = {}
        self.cursor = 0
        self.filled = 0

    def add(self, step: Mapping[str, torch.Tensor]) -> None:
        """One step of every environment: each field ``[envs, ...]``."""
        for k, v in step.items():
            if v.shape[0] != self.envs:
                raise ValueError(f"field {k!r} leads with {v.shape[0]}, the replay holds {self.envs} environments")
            if k not in self.held:
                self.held[k] = torch.zeros((self.capacity, self.envs) + tuple(v.shape[1:]), dtype=v.dtype, device=self.device)
            self.held[k][self.cursor] = v.to(self.device)
        self.cursor = (self.cursor + 1) % self.capacity
        self.filled = min(self.capacity, self.filled + 1)

    def extend(self, steps: Mapping[str, torch.Tensor]) -> None:
        """Several steps ``[T, envs, ...]`` in order."""
        T = next(iter(steps.values())).shape[0]
        for t in range(T):
            self.add({k: v[t] for k, v in steps.items()})

    def windows(self, length: int) -> int:
        return max(0, self.filled - length + 1)

    def sample(self, batch: int, length: int, generator: Optional[torch.Generator] = None) -> Dict[str, torch.Tensor]:
        """``batch`` windows of ``length`` consecutive steps, each from one environment: fields ``[batch, length, ...]``.  A window
        never spans the ring's seam (the oldest step follows the newest in memory, not in time)."""
        w = self.windows(length)
        if w <= 0:
            raise ValueError(f"the replay holds {self.filled} steps per environment, fewer than a window of {length}")
        first = torch.randint(0, w, (batch,), generator=generator)
        env = torch.randint(0, self.envs, (batch,), generator=generator)
        oldest = self.cursor if self.filled == self.capacity else 0
        t = (oldest + first[:, None] + torch.arange(length)[None]) % self.capacity            # [batch, length]
        t, env = t.to(self.device), env.to(self.device)
        return {k: v[t, env[:, None]] for k, v in self.held.items()}

    def state(self) -> Dict[str, object]:
        return {"held": self.held, "cursor": self.cursor, "filled": self.filled}

    def load_state(self, state) -> None:
        self.held, self.cursor, self.filled = dict(state["held"]), int(state["cursor"]), int(state["filled"])
