"""The gate race: a batch of quadrotors flies through a course of square gates; observations are the state relative to
the next gate and, optionally, the front camera's image (``dew_b200.rl.camera``).  Reference: src/dew/rl/flight.py
(``Scene``, ``Camera``, ``Renderer``), src/dew/rl/env.py."""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from .camera import Camera, gate_boxes, render
from .quadrotor import Quadrotor, QuadrotorState, quat_rotate


class GateRace:
    def __init__(self, batch: int, gates: int = 4, radius: float = 6.0, pillars: int = 3, camera: Optional[Camera] = None,
                 device="cpu", seed: int = 0, dt: float = 0.01, horizon: int = 1000):
        self.batch, self.device, self.dt, self.horizon = batch, torch.device(device), dt, horizon
        self.model, self.camera = Quadrotor(), camera
        g = torch.Generator().manual_seed(seed)
        ang = torch.arange(gates) * (2 * math.pi / gates)
        jitter = (torch.rand(batch, gates, 3, generator=g) - 0.5) * torch.tensor([1.0, 1.0, 0.6])
        centers = torch.stack([radius * torch.cos(ang), radius * torch.sin(ang), torch.full_like(ang, 1.5)], -1)[None] + jitter
        self.gate_centers = centers.to(self.device)                                  # [B, G, 3]
        self.gate_yaw = (ang + math.pi / 2)[None].expand(batch, gates).to(self.device).contiguous()
        self.boxes = gate_boxes(self.gate_centers, self.gate_yaw).reshape(batch, gates * 4, 10)
        pa = torch.rand(batch, pillars, generator=g) * 2 * math.pi
        pr = radius * (0.3 + 0.4 * torch.rand(batch, pillars, generator=g))
        self.cylinders = torch.stack([pr * torch.cos(pa), pr * torch.sin(pa), torch.full_like(pa, 0.25), torch.full_like(pa, 3.0),
                                      torch.full_like(pa, 0.5), torch.full_like(pa, 0.5), torch.full_like(pa, 0.55)], -1).to(self.device)
        self.generator = g
        self.reset()

    def reset(self) -> Dict[str, torch.Tensor]:
        self.state = self.model.reset(self.batch, self.device, self.generator, spread=1.0)
        self.previous = self.state
        self.next_gate = torch.zeros(self.batch, dtype=torch.long, device=self.device)
        self.steps = torch.zeros(self.batch, dtype=torch.long, device=self.device)
        return self.observe()

    def _target(self) -> torch.Tensor:
        return self.gate_centers[torch.arange(self.batch, device=self.device), self.next_gate % self.gate_centers.shape[1]]

    def cameras(self) -> torch.Tensor:
        """Shutter-open (previous step) and shutter-close (now) camera poses ``[B, 2, 12]`` looking along the body x axis."""
        rows = []
        for s in (self.previous, self.state):
            fwd = quat_rotate(s.quaternion, torch.tensor([1.0, 0, 0], device=self.device).expand(self.batch, 3))
            left = quat_rotate(s.quaternion, torch.tensor([0.0, 1, 0], device=self.device).expand(self.batch, 3))
            up = quat_rotate(s.quaternion, torch.tensor([0.0, 0, 1], device=self.device).expand(self.batch, 3))
            rows.append(torch.cat([s.position, -left, -up, fwd], -1))
        return torch.stack(rows, 1)

    def observe(self) -> Dict[str, torch.Tensor]:
        s = self.state
        obs = {"state": torch.cat([self._target() - s.position, s.velocity, s.quaternion, s.rates], -1)}
        if self.camera is not None:
            obs["image"] = render(self.cameras(), self.boxes, self.cylinders, self.camera)
        return obs

    def step(self, action: torch.Tensor) -> Tuple[Dict[str, torch.Tensor], torch.Tensor, torch.Tensor]:
        before = (self._target() - self.state.position).norm(dim=-1)
        self.previous = self.state
        self.state = self.model.step(self.state, action, self.dt)
        self.steps += 1
        after = (self._target() - self.state.position).norm(dim=-1)
        passed = after < 0.5
        reward = (before - after) + 10.0 * passed.float() - 1e-3 * action.pow(2).sum(-1)
        self.next_gate = self.next_gate + passed.long()
        crashed = (self.state.position[:, 2] < 0.05) | (self.state.position.norm(dim=-1) > 30)
        done = crashed | (self.steps >= self.horizon)
        reward = reward - 5.0 * crashed.float()
        return self.observe(), reward, done
