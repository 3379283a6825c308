"""Batched quadrotor rigid-body dynamics (position, velocity, unit quaternion, body rates; four rotor thrusts in),
integrated with semi-implicit Euler.  Reference: src/dew/rl/quadrotor.py (305 lines), src/dew/rl/simulator.py."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class QuadrotorState:
    position: torch.Tensor      # [B, 3]
    velocity: torch.Tensor      # [B, 3]
    quaternion: torch.Tensor    # [B, 4] (w, x, y, z), body -> world
    rates: torch.Tensor         # [B, 3] body angular velocity


def quat_rotate(q, v):
    w, u = q[..., :1], q[..., 1:]
    t = 2 * torch.cross(u, v, dim=-1)
    return v + w * t + torch.cross(u, t, dim=-1)


def quat_multiply(a, b):
    aw, ax, ay, az = a.unbind(-1)
    bw, bx, by, bz = b.unbind(-1)
    return torch.stack([aw * bw - ax * bx - ay * by - az * bz, aw * bx + ax * bw + ay * bz - az * by,
                        aw * by - ax * bz + ay * bw + az * bx, aw * bz + ax * by - ay * bx + az * bw], -1)


class Quadrotor:
    def __init__(self, mass=0.8, arm=0.12, inertia=(4e-3, 4e-3, 7e-3), thrust_max=6.0, torque_ratio=0.016, drag=0.1, gravity=9.81):
        self.mass, self.arm, self.thrust_max, self.kappa, self.drag, self.g = mass, arm, thrust_max, torque_ratio, drag, gravity
        self.inertia = torch.tensor(inertia)

    def reset(self, batch: int, device="cpu", generator=None, spread: float = 0.0) -> QuadrotorState:
        pos = torch.zeros(batch, 3, device=device)
        if spread:
            pos = pos + spread * (torch.rand(batch, 3, generator=generator).to(device) - 0.5)
        pos[:, 2] = pos[:, 2].abs() + 1.0
        q = torch.zeros(batch, 4, device=device); q[:, 0] = 1
        return QuadrotorState(pos, torch.zeros(batch, 3, device=device), q, torch.zeros(batch, 3, device=device))

    def step(self, s: QuadrotorState, action: torch.Tensor, dt: float = 0.01) -> QuadrotorState:
        """``action [B, 4]`` in [-1, 1]: rotor commands (front-left, front-right, rear-right, rear-left)."""
        f = (action.clamp(-1, 1) + 1) * 0.5 * self.thrust_max                      # per-rotor thrust, N
        a = self.arm / 2 ** 0.5
        torque = torch.stack([a * (f[:, 0] - f[:, 1] - f[:, 2] + f[:, 3]), a * (-f[:, 0] - f[:, 1] + f[:, 2] + f[:, 3]),
                              self.kappa * (f[:, 0] - f[:, 1] + f[:, 2] - f[:, 3])], -1)
        I = self.inertia.to(f.device)
        rates = s.rates + dt * (torque - torch.cross(s.rates, I * s.rates, dim=-1)) / I
        dq = torch.cat([torch.zeros_like(rates[:, :1]), rates], -1)
        q = s.quaternion + 0.5 * dt * quat_multiply(s.quaternion, dq)
        q = q / q.norm(dim=-1, keepdim=True)
        thrust = torch.zeros_like(s.velocity); thrust[:, 2] = f.sum(-1)
        acc = quat_rotate(q, thrust) / self.mass - self.drag * s.velocity
        acc[:, 2] = acc[:, 2] - self.g
        vel = s.velocity + dt * acc
        return QuadrotorState(s.position + dt * vel, vel, q, rates)
