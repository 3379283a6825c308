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


# ================================================================================================ the racing drone
# A five-inch FPV racer as the drone-racing literature models it (Kaufmann, Bauersfeld, Scaramuzza, arXiv 2202.10796, Eq 1-3 and
# Table II; Flightmare's and L2F's racer configuration; SkyDreamer, arXiv 2510.14783, Sec II-D and Tables II-III): a rigid body
# under four rotors in an X, thrust c_l w^2 and yaw torque c_d w^2 per rotor, rotor speeds following their steady speeds through
# a first-order lag, a battery whose voltage sags under load, a Betaflight-style rate controller run every physics step, rotor /
# quadratic / vertical drag, ground effect, a constant disturbance per episode and noised duties.  Every parameter is drawn per
# episode, its spread about nominal scaled by ``ramp`` (0: the nominal drone, no disturbance; 1: the full randomisation).
# World frame: x forward, y left, z up; body frame: forward, left, up.  Reference: src/dew/rl/quadrotor.py (``Quadrotor``,
# ``Body``, ``Flight``, ``drawn_body``, ``rotation``, ``hovering``, ``duties``, ``flown``).
import math
from dataclasses import field
from typing import Dict, Tuple

ARM = 0.17 * 0.5 ** 0.5                                                   # a rotor's offset along x and y: a 0.17 m arm in an X
POSITIONS = ((ARM, -ARM), (-ARM, -ARM), (-ARM, ARM), (ARM, ARM))          # front right, rear right, rear left, front left
SPINS = (-1.0, 1.0, -1.0, 1.0)                                            # each rotor's yaw torque's sign
GRAVITY = 9.81


@dataclass(frozen=True)
class Racer:
    mass: float = 0.73
    mass_spread: float = 0.04
    inertia: Tuple[float, float, float] = (2.38e-3, 2.0e-3, 4.09e-3)
    inertia_spread: float = 0.1
    thrust_coefficient: float = 1.563e-6          # N s^2
    thrust_spread: float = 0.1
    drag_coefficient: float = 1.909e-8            # N m s^2
    drag_spread: float = 0.1
    top_speed: float = 3700.0                     # rad/s
    top_speed_spread: float = 0.05
    idle_speed: float = 300.0
    motor_lag: Tuple[float, float] = (0.033, 0.040)
    rotor_drag: float = 5.37e-5                   # N s / (m rad)
    quadratic_drag: Tuple[float, float] = (4.10e-3, 1.51e-2)
    vertical_drag: float = 0.15                   # N s / m
    drag_spread_air: float = 0.2
    ground_effect: Tuple[float, float] = (0.75, 1.0)
    rotor_radius: float = 0.0635
    cells: int = 6
    full_voltage: float = 4.2
    charged: Tuple[float, float] = (3.9, 4.2)     # each cell's open-circuit voltage at the start
    discharge: float = 0.6                        # volts a cell loses over the pack's charge
    resistance: Tuple[float, float] = (4.5e-3, 9.0e-3)
    capacity: float = 1.3                         # Ah
    efficiency: float = 0.6                       # shaft power over electrical power (an assumption)
    bias_force: float = 2.0                       # m/s^2 at most
    bias_moment: float = 2.0                      # rad/s^2 at most
    duty_noise: float = 0.2
    rate_gain: float = 100.0
    rate_damping: float = 2.0
    substeps: int = 4

    @property
    def hover_speed(self) -> float:
        return math.sqrt(self.mass * GRAVITY / (4 * self.thrust_coefficient))


Body = Dict[str, torch.Tensor]
Flight = Dict[str, torch.Tensor]


def _uniform(g, n, low, high, device):
    return (low + (high - low) * torch.rand(n, generator=g)).to(device)


def _about(g, n, nominal, spread, ramp, device, width=()):
    shape = (n,) + tuple(width)
    return (torch.as_tensor(nominal, dtype=torch.float32) * (1 + spread * ramp * (2 * torch.rand(shape, generator=g) - 1))).to(device)


def drawn_body(racer: Racer, key: int, count: int, ramp: float = 1.0, device="cpu") -> Body:
    g = torch.Generator().manual_seed(int(key) & 0x7FFFFFFF)
    mid = lambda lo_hi: 0.5 * (lo_hi[0] + lo_hi[1])
    around = lambda lo_hi: _uniform(g, count, mid(lo_hi) - ramp * (mid(lo_hi) - lo_hi[0]), mid(lo_hi) + ramp * (lo_hi[1] - mid(lo_hi)), device)
    direction = torch.randn(count, 3, generator=g)
    direction = direction / direction.norm(dim=-1, keepdim=True).clamp_min(1e-9)
    moment_dir = torch.randn(count, 3, generator=g)
    moment_dir = moment_dir / moment_dir.norm(dim=-1, keepdim=True).clamp_min(1e-9)
    mass = _about(g, count, racer.mass, racer.mass_spread, ramp, device)
    inertia = _about(g, count, racer.inertia, racer.inertia_spread, ramp, device, (3,))
    return {"mass": mass, "inertia": inertia,
            "thrust_coefficient": _about(g, count, racer.thrust_coefficient, racer.thrust_spread, ramp, device),
            "drag_coefficient": _about(g, count, racer.drag_coefficient, racer.drag_spread, ramp, device),
            "top_speed": _about(g, count, racer.top_speed, racer.top_speed_spread, ramp, device),
            "motor_lag": around(racer.motor_lag),
            "rotor_drag": _about(g, count, racer.rotor_drag, racer.drag_spread_air, ramp, device),
            "quadratic_drag": _about(g, count, racer.quadratic_drag, racer.drag_spread_air, ramp, device, (2,)),
            "vertical_drag": _about(g, count, racer.vertical_drag, racer.drag_spread_air, ramp, device),
            "ground_effect": around(racer.ground_effect) * (ramp > 0),
            "charged": _uniform(g, count, racer.charged[1] - ramp * (racer.charged[1] - racer.charged[0]), racer.charged[1], device),
            "resistance": around(racer.resistance),
            "force": (direction * torch.rand(count, 1, generator=g) * racer.bias_force * ramp).to(device) * mass[:, None],
            "moment": (moment_dir * torch.rand(count, 1, generator=g) * racer.bias_moment * ramp).to(device) * inertia,
            "duty_noise": torch.full((count,), racer.duty_noise * ramp, device=device)}


def rotation(q: torch.Tensor) -> torch.Tensor:
    """Body-to-world rotation matrices ``[..., 3, 3]`` of unit quaternions (w, x, y, z)."""
    w, x, y, z = q.unbind(-1)
    return torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y),
                        2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x),
                        2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], -1).reshape(*q.shape[:-1], 3, 3)


def quaternion_of(yaw: torch.Tensor, pitch=None, roll=None) -> torch.Tensor:
    """Unit quaternions of a yaw, then a pitch, then a roll."""
    zero = torch.zeros_like(yaw)
    pitch = zero if pitch is None else pitch
    roll = zero if roll is None else roll
    cy, sy, cp, sp, cr, sr = torch.cos(yaw / 2), torch.sin(yaw / 2), torch.cos(pitch / 2), torch.sin(pitch / 2), torch.cos(roll / 2), torch.sin(roll / 2)
    return torch.stack([cr * cp * cy + sr * sp * sy, sr * cp * cy - cr * sp * sy, cr * sp * cy + sr * cp * sy, cr * cp * sy - sr * sp * cy], -1)


def voltage(racer: Racer, body: Body, speed: torch.Tensor, used: torch.Tensor) -> torch.Tensor:
    """The pack's voltage under the rotors' load: open-circuit voltage fallen with the charge used, sagged by the internal
    resistance times the current (the rotors' shaft power over the efficiency, over the voltage - solved as a quadratic)."""
    open_circuit = racer.cells * (body["charged"] - racer.discharge * used / racer.capacity)
    power = (body["drag_coefficient"][:, None] * speed ** 3).sum(-1) / racer.efficiency
    r = racer.cells * body["resistance"]
    # V = E - R P / V  ->  V^2 - E V + R P = 0, the upper root; a load past the pack's ability floors the root at E / 2
    disc = (open_circuit ** 2 - 4 * r * power).clamp_min(0)
    return 0.5 * (open_circuit + disc.sqrt())


def hovering(racer: Racer, body: Body, position: torch.Tensor, orientation: torch.Tensor) -> Flight:
    n = position.shape[0]
    w = torch.sqrt(body["mass"] * GRAVITY / (4 * body["thrust_coefficient"]))
    zeros = torch.zeros(n, 3, device=position.device)
    return {"position": position, "velocity": zeros, "orientation": orientation, "angular_velocity": zeros.clone(),
            "speed": w[:, None].expand(n, 4).contiguous(), "used": torch.zeros(n, device=position.device), "rate_before": zeros.clone()}


def _mixer(racer: Racer) -> torch.Tensor:
    """Rotor thrusts from (collective, torque x, torque y, torque z): the inverse of the X configuration's allocation."""
    ratio = racer.drag_coefficient / racer.thrust_coefficient
    rows = [[1.0] * 4, [y for _, y in POSITIONS], [-x for x, _ in POSITIONS], [s * ratio for s in SPINS]]
    return torch.linalg.inv(torch.tensor(rows, dtype=torch.float64)).float()


def duties(racer: Racer, flight: Flight, collective: torch.Tensor, rates: torch.Tensor, dt: float) -> torch.Tensor:
    """The flight controller's duties ``[N, 4]`` in [0, 1] for a collective thrust (N) and body rates (rad/s): a PD loop on the
    body rates to angular accelerations, times the nominal inertia, mixed with the collective into rotor thrusts, then each
    rotor's duty from the nominal thrust map."""
    w = flight["angular_velocity"]
    accel = racer.rate_gain * (rates - w) - racer.rate_damping * (w - flight["rate_before"]) / dt
    torque = accel * torch.tensor(racer.inertia, device=w.device)
    wrench = torch.cat([collective[:, None], torque], -1)
    thrusts = (wrench @ _mixer(racer).to(w.device).t()).clamp_min(0)
    speed = torch.sqrt(thrusts / racer.thrust_coefficient)
    return (speed / racer.top_speed).clamp(0, 1)


def flown(racer: Racer, body: Body, flight: Flight, collective: torch.Tensor, rates: torch.Tensor, hz: float, key: int = 0
          ) -> Tuple[Flight, torch.Tensor]:
    """The drone after a control step of ``1 / hz`` seconds under a collective thrust (N) and body rates (rad/s), and its path
    ``[N, substeps + 1, 3]`` (its positions before the step and after each physics step)."""
    dev = flight["position"].device
    n = flight["position"].shape[0]
    dt = 1.0 / (hz * racer.substeps)
    g = torch.Generator().manual_seed(int(key) & 0x7FFFFFFF)
    noise = (body["duty_noise"][:, None] * (2 * torch.rand(n, 4, generator=g).to(dev) - 1))
    pos_xy = torch.tensor(POSITIONS, device=dev)
    spins = torch.tensor(SPINS, device=dev)
    f = dict(flight)
    path = [f["position"]]
    for _ in range(racer.substeps):
        duty = (duties(racer, f, collective, rates, dt) + noise * 0.05).clamp(0, 1)
        volts = voltage(racer, body, f["speed"], f["used"])
        steady = (duty * body["top_speed"][:, None] * (volts / (racer.cells * racer.full_voltage))[:, None]).clamp_min(racer.idle_speed)
        speed = f["speed"] + (steady - f["speed"]) * (1 - torch.exp(-dt / body["motor_lag"]))[:, None]
        height = f["position"][:, 2].clamp_min(racer.rotor_radius)
        lift = 1.0 / (1.0 - body["ground_effect"] * (racer.rotor_radius / (4 * height)) ** 2).clamp_min(0.5)
        thrust = body["thrust_coefficient"][:, None] * speed ** 2 * lift[:, None]                         # [N, 4]
        R = rotation(f["orientation"])
        v_body = torch.einsum("nij,ni->nj", R, f["velocity"])                                              # R^T v
        drag = torch.stack([-(body["rotor_drag"] * speed.sum(-1)) * v_body[:, 0] - body["quadratic_drag"][:, 0] * v_body[:, 0] * v_body[:, 0].abs(),
                            -(body["rotor_drag"] * speed.sum(-1)) * v_body[:, 1] - body["quadratic_drag"][:, 1] * v_body[:, 1] * v_body[:, 1].abs(),
                            -body["vertical_drag"] * v_body[:, 2]], -1)
        force_body = drag + torch.stack([torch.zeros(n, device=dev), torch.zeros(n, device=dev), thrust.sum(-1)], -1)
        accel = torch.einsum("nij,nj->ni", R, force_body) / body["mass"][:, None] + body["force"] / body["mass"][:, None]
        accel = accel - torch.tensor([0.0, 0.0, GRAVITY], device=dev)
        torque = torch.stack([(thrust * pos_xy[:, 1]).sum(-1), -(thrust * pos_xy[:, 0]).sum(-1),
                              (body["drag_coefficient"][:, None] * speed ** 2 * spins).sum(-1)], -1) + body["moment"]
        w = f["angular_velocity"]
        w_new = w + dt * (torque - torch.cross(w, body["inertia"] * w, dim=-1)) / body["inertia"]
        dq = torch.cat([torch.zeros(n, 1, device=dev), w_new], -1)
        q = f["orientation"] + 0.5 * dt * quat_multiply(f["orientation"], dq)
        q = q / q.norm(dim=-1, keepdim=True)
        vel = f["velocity"] + dt * accel
        current = (body["drag_coefficient"][:, None] * speed ** 3).sum(-1) / racer.efficiency / volts.clamp_min(1.0)
        f = {"position": f["position"] + dt * vel, "velocity": vel, "orientation": q, "angular_velocity": w_new, "speed": speed,
             "used": f["used"] + current * dt / 3600.0, "rate_before": w}
        path.append(f["position"])
    return f, torch.stack(path, 1)
