"""First-person drone gate racing: a batch of drones' races as an ``Env`` (``FlightEnv``), flown by ``quadrotor``'s racing physics,
and the same races seen through the ray-cast camera as a host-stepped ``Simulator`` (``GateRace``).

The reward is the one drone-racing RL has converged on (Kaufmann et al., Nature 2023, Eq 8; Song et al., Sci. Robot. 2023, Eq 5;
SkyDreamer, arXiv 2510.14783, Sec II-C): each step the progress made toward the next gate's centre, less a cost on the body
rates and on the action's change; a bonus on passing a gate, larger when passed centred; a reward for the camera's optical
axis pointing at the next gate (``scale * exp(-sharpness * angle^4)``); a penalty and the episode's end on a crash (the gate's
frame, the ground, a pillar, the ceiling, or straying ``miss_radius`` past the gate's plane without passing it).

A course is drawn per episode from a family (``loop``: gates on a jittered circle; ``chain``: a track of random turns and
climbs; ``figure8``; ``layout``: a named fixed layout, jittered), with up to ``obstacles`` pillars, some on the racing line.
``difficulty`` in [0, 1] scales jitter, turns and obstacles; ``ramp`` scales the drone's randomisation (``quadrotor.drawn_body``).
Actions ``[N, 4]`` in [-1, 1]: the throttle (below zero a share of the hover thrust, above it a share of the span from hover to
the most the nominal drone lifts) and three body rates as shares of the drone's rate limit, taken by the flight controller after
the drone's command latency.  Observations are the privileged views asked for: ``state [13]``, ``gates [24]`` (the next two
gates' opening corners in the body frame), ``airframe [6]``, ``obstacles [4 * NEAREST]``, ``action [4]``, ``progress [3]``.

Reference: src/dew/rl/flight.py (``Racing``, ``Course``, ``Race``, ``drawn_course``, ``facings``, ``gate_axes``, ``commanded``,
``delayed``, ``struck``, ``raced``, ``looking``, ``corners``, ``nearest``, ``privileged``, ``FlightEnv``, ``Scene``, ``GateRace``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional, Sequence, Tuple

import torch

from .camera import Camera, gate_boxes, render
from .env import Env, TimeStep, chosen, tree_map
from .quadrotor import (GRAVITY, Racer, drawn_body, flown, hovering, quaternion_of, rotation)
from .simulator import Branching, Simulator

FAMILIES = ("layout", "loop", "chain", "figure8")
GATES = 12
OBSTACLES = 6
NEAREST = 3
VIEWS = ("state", "gates", "airframe", "obstacles", "action", "progress")
LAYOUTS: Dict[str, Tuple[Tuple[float, float, float], ...]] = {
    # an oval and a stacked pair of turns (a descending half turn under a climbing one)
    "oval": ((6, 0, 1.5), (12, 3, 1.5), (12, 9, 2.0), (6, 12, 1.5), (0, 9, 1.5), (0, 3, 2.0)),
    "stack": ((6, 0, 1.5), (12, 0, 3.5), (16, 4, 3.5), (12, 8, 3.5), (12, 8, 1.5), (6, 4, 1.5), (0, 4, 2.0)),
}


@dataclass(frozen=True)
class Racing:
    families: Tuple[Tuple[str, float], ...] = (("loop", 0.4), ("chain", 0.6))
    layouts: Tuple[str, ...] = tuple(LAYOUTS)
    jitter: Tuple[float, float] = (1.5, 0.75)
    gates: Tuple[int, int] = (4, 8)
    spacing: Tuple[float, float] = (5.0, 9.0)
    obstacles: int = OBSTACLES
    on_line: float = 0.3
    hz: float = 60.0
    episode_seconds: float = 25.0
    opening: float = 1.5
    frame: float = 0.25
    depth: float = 0.1
    radius: float = 0.2
    progress_scale: float = 1.0
    rate_cost: float = 1.0 / 100
    smoothness_cost: float = 0.005
    gate_bonus: float = 6.0
    perception_scale: float = 0.02
    perception_sharpness: float = 10.0
    crash_penalty: float = 10.0
    miss_radius: float = 3.0
    ceiling: float = 25.0
    bounds: float = 60.0
    rate_limit: float = 10.0
    rate_spread: float = 0.2
    latency: Tuple[float, float] = (0.01, 0.06)
    uptilt: float = 30.0
    flying_share: float = 0.3
    start_speed: float = 6.0
    racer: Racer = field(default_factory=Racer)

    @property
    def episode_steps(self) -> int:
        return int(round(self.episode_seconds * self.hz))

    @property
    def max_delay(self) -> int:
        return int(math.ceil(self.latency[1] * self.hz))


# ------------------------------------------------------------------------------------------------ courses
def facings(centres: torch.Tensor, count: torch.Tensor, closed: torch.Tensor) -> torch.Tensor:
    """Each gate's facing ``[N, G]``: the yaw of the level line from the gate before it to the gate after it - wrapping round on a
    closed course, on an open one the first gate's from itself and the last's to itself."""
    N, G, _ = centres.shape
    idx = torch.arange(G, device=centres.device)[None].expand(N, G)
    c = count[:, None]
    before = torch.where(closed[:, None], (idx - 1) % c, (idx - 1).clamp_min(0))
    after = torch.where(closed[:, None], (idx + 1) % c, torch.minimum(idx + 1, c - 1))
    gather = lambda i: centres.gather(1, i.clamp(0, G - 1)[..., None].expand(N, G, 3))
    d = gather(after) - gather(before)
    return torch.atan2(d[..., 1], d[..., 0])


def gate_axes(facing: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """A gate's normal (its passing direction) and its left, both level, from its facing."""
    zero = torch.zeros_like(facing)
    return torch.stack([torch.cos(facing), torch.sin(facing), zero], -1), torch.stack([-torch.sin(facing), torch.cos(facing), zero], -1)


def drawn_course(racing: Racing, key: int, count: int, difficulty: float = 1.0, device="cpu") -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(int(key) & 0x7FFFFFFF)
    names = [n for n, _ in racing.families]
    weights = torch.tensor([w for _, w in racing.families], dtype=torch.float32)
    family = torch.multinomial(weights / weights.sum(), count, replacement=True, generator=g)
    lo, hi = racing.gates
    n_gates = torch.randint(lo, hi + 1, (count,), generator=g)
    centres = torch.zeros(count, GATES, 3)
    closed = torch.zeros(count, dtype=torch.bool)
    jx, jz = racing.jitter
    for i in range(count):
        fam = names[int(family[i])]
        k = int(n_gates[i])
        u = lambda *s: torch.rand(*s, generator=g)
        if fam == "loop":
            radius = 0.5 * k * float(racing.spacing[0] + (racing.spacing[1] - racing.spacing[0]) * u(1)) / math.pi
            ang = torch.arange(k) * (2 * math.pi / k)
            r = radius * (1 + 0.25 * difficulty * (2 * u(k) - 1))
            pts = torch.stack([r * torch.cos(ang), r * torch.sin(ang), 1.5 + jz * difficulty * (2 * u(k) - 1).clamp_min(-0.6)], -1)
            closed[i] = True
        elif fam == "figure8":
            k = max(k, 6) // 2 * 2
            ang = torch.arange(k) * (2 * math.pi / k)
            a = 0.35 * k * racing.spacing[0] / 2
            pts = torch.stack([a * torch.sin(ang), a * torch.sin(ang) * torch.cos(ang), 1.5 + 1.0 * difficulty * torch.cos(ang) ** 2], -1)
            closed[i] = True
        elif fam == "layout":
            layout = LAYOUTS[racing.layouts[int(torch.randint(0, len(racing.layouts), (1,), generator=g))]]
            pts = torch.tensor(layout, dtype=torch.float32)
            k = pts.shape[0]
            pts = pts + difficulty * (2 * u(k, 3) - 1) * torch.tensor([jx, jx, jz])
            closed[i] = True
        else:                                                            # chain: a track of random turns and climbs
            heading = float(2 * math.pi * u(1))
            p = torch.zeros(3)
            p[2] = 1.5
            out = []
            for _ in range(k):
                step = float(racing.spacing[0] + (racing.spacing[1] - racing.spacing[0]) * u(1))
                heading += float((2 * u(1) - 1) * (0.35 + 0.9 * difficulty))
                p = p + torch.tensor([step * math.cos(heading), step * math.sin(heading), float((2 * u(1) - 1) * jz * 2 * difficulty)])
                p[2] = p[2].clamp(1.0, 6.0)
                out.append(p.clone())
            pts = torch.stack(out)
        pts[:, 2] = pts[:, 2].clamp_min(racing.opening / 2 + racing.frame + 0.2)
        n_gates[i] = k
        centres[i, :k] = pts
        centres[i, k:] = pts[-1]
    facing = facings(centres, n_gates, closed)
    # pillars: some on the racing line between two gates, the rest scattered near the course
    n_obs = torch.round(racing.obstacles * difficulty * torch.rand(count, generator=g)).long()
    obstacles = torch.zeros(count, OBSTACLES, 4)                                                 # x, y, radius, height
    for i in range(count):
        k = int(n_gates[i])
        for o in range(min(int(n_obs[i]), OBSTACLES)):
            a = int(torch.randint(0, k - 1 if k > 1 else 1, (1,), generator=g))
            t = float(0.35 + 0.3 * torch.rand(1, generator=g))
            mid = centres[i, a] * (1 - t) + centres[i, min(a + 1, k - 1)] * t
            on_line = float(torch.rand(1, generator=g)) < racing.on_line
            off = (2 * torch.rand(2, generator=g) - 1) * (0.6 if on_line else 4.0)
            if not on_line:
                off = off + torch.sign(off) * 1.5
            radius = float(0.15 + 0.35 * torch.rand(1, generator=g))
            obstacles[i, o] = torch.tensor([float(mid[0] + off[0]), float(mid[1] + off[1]), radius, radius * float([6.0, 12.0, 24.0][o % 3])])
    to = lambda x: x.to(device)
    return {"centres": to(centres), "facing": to(facing), "count": to(n_gates), "closed": to(closed), "family": to(family), "obstacles": to(obstacles)}


# ------------------------------------------------------------------------------------------------ commands
def commanded(racing: Racing, body, rate_limit: torch.Tensor, action: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """An action ``[N, 4]`` in [-1, 1] as a collective thrust (N) and body rates (rad/s): below zero the throttle is a share of the
    hover thrust, above it a share of the span from the hover to the nominal drone's most."""
    a = action.clamp(-1, 1)
    r = racing.racer
    hover = r.mass * GRAVITY
    most = 4 * r.thrust_coefficient * r.top_speed ** 2
    throttle = a[:, 0]
    collective = torch.where(throttle < 0, hover * (1 + throttle), hover + throttle * (most - hover))
    return collective, a[:, 1:] * rate_limit[:, None]


def delayed(pending: torch.Tensor, command: torch.Tensor, delay: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``pending [N, D + 1, C]`` newest first with ``command`` pushed, and the command ``delay [N]`` steps old."""
    pending = torch.cat([command[:, None], pending[:, :-1]], 1)
    taken = pending.gather(1, delay.clamp(0, pending.shape[1] - 1)[:, None, None].expand(-1, 1, pending.shape[-1])).squeeze(1)
    return pending, taken


# ------------------------------------------------------------------------------------------------ collisions
def struck(racing: Racing, path: torch.Tensor, centre: torch.Tensor, facing: torch.Tensor, obstacles: torch.Tensor
           ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Whether each drone's path through a step ``[N, S + 1, 3]`` (straight segments between physics steps) crashed, passed the
    gate it heads for, and how far from the opening's centre it crossed (as a share of the half opening; zero where it did not)."""
    N, S1, _ = path.shape
    normal, left = gate_axes(facing)
    up = torch.tensor([0.0, 0.0, 1.0], device=path.device).expand(N, 3)
    rel = path - centre[:, None]
    along = (rel * normal[:, None]).sum(-1)                                                    # [N, S + 1]
    a0, a1 = along[:, :-1], along[:, 1:]
    crossing = (a0 < 0) & (a1 >= 0)
    t = (-a0 / (a1 - a0).clamp_min(1e-9)).clamp(0, 1)
    point = rel[:, :-1] + (rel[:, 1:] - rel[:, :-1]) * t[..., None]
    y = (point * left[:, None]).sum(-1).abs()
    z = (point * up[:, None]).sum(-1).abs()
    half = racing.opening / 2
    inside = (y <= half - racing.radius) & (z <= half - racing.radius)
    on_frame = ~inside & (y <= half + racing.frame + racing.radius) & (z <= half + racing.frame + racing.radius)
    passed_seg = crossing & inside
    passed = passed_seg.any(1)
    offset = (torch.maximum(y, z) / half * passed_seg).sum(1) / passed_seg.sum(1).clamp_min(1)
    # the frame from behind too: a crossing in either direction through the frame's bars
    backward = (a0 >= 0) & (a1 < 0)
    hit_frame = ((crossing | backward) & on_frame).any(1)
    ground = (path[..., 2] < racing.radius).any(1)
    high = (path[..., 2] > racing.ceiling).any(1) | (path[..., :2].abs() > racing.bounds).any(-1).any(1)
    # pillars: the horizontal distance from each path point to each pillar's axis, below its top
    d = (path[:, :, None, :2] - obstacles[:, None, :, :2]).norm(dim=-1)                          # [N, S + 1, O]
    live = obstacles[:, None, :, 2] > 0
    pillar = (live & (d < obstacles[:, None, :, 2] + racing.radius) & (path[:, :, None, 2] < obstacles[:, None, :, 3])).any(-1).any(-1)
    return hit_frame | ground | high | pillar, passed & ~hit_frame, offset


def looking(racing: Racing, flight, point: torch.Tensor) -> torch.Tensor:
    """The angle between the camera's optical axis (the body's forward tilted up by the uptilt) and the direction to ``point``."""
    R = rotation(flight["orientation"])
    tilt = math.radians(racing.uptilt)
    axis = R @ torch.tensor([math.cos(tilt), 0.0, math.sin(tilt)], device=point.device)
    to = point - flight["position"]
    to = to / to.norm(dim=-1, keepdim=True).clamp_min(1e-9)
    return torch.acos((axis * to).sum(-1).clamp(-1, 1))


def corners(racing: Racing, course, flight, target: torch.Tensor, ahead: int = 2) -> torch.Tensor:
    """The corners of the openings of the gate headed for and the ``ahead - 1`` after it, in the body frame ``[N, 12 * ahead]``
    (on an open track the last gate stands in for any beyond it)."""
    N = target.shape[0]
    R = rotation(flight["orientation"])
    out = []
    half = racing.opening / 2
    for k in range(ahead):
        idx = target + k
        idx = torch.where(course["closed"], idx % course["count"], torch.minimum(idx, course["count"] - 1))
        c = course["centres"].gather(1, idx[:, None, None].expand(N, 1, 3)).squeeze(1)
        f = course["facing"].gather(1, idx[:, None]).squeeze(1)
        _, left = gate_axes(f)
        up = torch.tensor([0.0, 0.0, 1.0], device=c.device)
        for sy, sz in ((1, 1), (-1, 1), (-1, -1), (1, -1)):
            world = c + sy * half * left + sz * half * up - flight["position"]
            out.append(torch.einsum("nij,ni->nj", R, world))
    return torch.cat(out, -1)


def nearest(racing: Racing, course, flight) -> torch.Tensor:
    """The ``NEAREST`` live pillars nearest the drone: each axis's offset in the body frame (at the drone's height, held within
    the pillar) and its radius ``[N, 4 * NEAREST]``; an absent one is zeros."""
    obs = course["obstacles"]
    N = obs.shape[0]
    R = rotation(flight["orientation"])
    p = flight["position"]
    d = (obs[..., :2] - p[:, None, :2]).norm(dim=-1)
    d = torch.where(obs[..., 2] > 0, d, torch.full_like(d, float("inf")))
    order = d.argsort(1)[:, :NEAREST]
    pick = obs.gather(1, order[..., None].expand(N, NEAREST, 4))
    live = pick[..., 2] > 0
    height = torch.minimum(p[:, None, 2].expand(N, NEAREST), pick[..., 3])
    world = torch.stack([pick[..., 0] - p[:, None, 0], pick[..., 1] - p[:, None, 1], height - p[:, None, 2]], -1)
    body = torch.einsum("nij,nki->nkj", R, world)
    return (torch.cat([body, pick[..., 2:3]], -1) * live[..., None]).reshape(N, 4 * NEAREST)


# ------------------------------------------------------------------------------------------------ the environment
class FlightEnv(Env):
    action_size = 4

    def __init__(self, racing: Racing = Racing(), views: Sequence[str] = ("state", "gates", "action"), difficulty: float = 1.0,
                 ramp: float = 1.0, device="cpu"):
        unknown = set(views) - set(VIEWS)
        if unknown:
            raise ValueError(f"views {sorted(unknown)} are none of {VIEWS}")
        self.racing, self.views, self.difficulty, self.ramp, self.device = racing, tuple(views), difficulty, ramp, torch.device(device)

    # -- helpers
    def _gate(self, course, index: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        N = index.shape[0]
        idx = torch.where(course["closed"], index % course["count"], torch.minimum(index, course["count"] - 1))
        return (course["centres"].gather(1, idx[:, None, None].expand(N, 1, 3)).squeeze(1), course["facing"].gather(1, idx[:, None]).squeeze(1))

    def observe(self, state) -> Dict[str, torch.Tensor]:
        f, course = state["flight"], state["course"]
        out = {}
        if "state" in self.views:
            out["state"] = torch.cat([f["position"], f["velocity"], f["orientation"], f["angular_velocity"]], -1)
        if "gates" in self.views:
            out["gates"] = corners(self.racing, course, f, state["target"])
        if "airframe" in self.views:
            r, b = self.racing.racer, state["body"]
            lift = 4 * b["thrust_coefficient"] * b["top_speed"] ** 2 * (b["charged"] / r.full_voltage) ** 2 / (b["mass"] * GRAVITY)
            nominal = 4 * r.thrust_coefficient * r.top_speed ** 2 / (r.mass * GRAVITY)
            out["airframe"] = torch.stack([lift / nominal, state["rate_limit"] / self.racing.rate_limit, b["motor_lag"] / (0.5 * sum(r.motor_lag)),
                                           state["delay"].float() / max(1, self.racing.max_delay), b["mass"] / r.mass,
                                           b["rotor_drag"] / r.rotor_drag], -1)
        if "obstacles" in self.views:
            out["obstacles"] = nearest(self.racing, course, f)
        if "action" in self.views:
            out["action"] = state["last_action"]
        if "progress" in self.views:
            out["progress"] = torch.stack([state["passed"].float(), state["distance"], state["steps"].float() / self.racing.episode_steps], -1)
        return out

    def reset(self, key: int, count: int):
        rc, dev = self.racing, self.device
        g = torch.Generator().manual_seed((int(key) * 7919 + 13) & 0x7FFFFFFF)
        course = drawn_course(rc, key, count, self.difficulty, dev)
        body = drawn_body(rc.racer, int(key) + 1, count, self.ramp, dev)
        first, facing0 = course["centres"][:, 0], course["facing"][:, 0]
        normal, left = gate_axes(facing0)
        back = (3.0 + 3.0 * torch.rand(count, generator=g)).to(dev)
        side = ((2 * torch.rand(count, generator=g) - 1) * 1.0 * self.difficulty).to(dev)
        position = first - normal * back[:, None] + left * side[:, None]
        position[:, 2] = (first[:, 2] + ((2 * torch.rand(count, generator=g) - 1) * 0.5 * self.difficulty).to(dev)).clamp_min(0.6)
        yaw = facing0 + ((2 * torch.rand(count, generator=g) - 1) * 0.5 * self.difficulty).to(dev)
        flight = hovering(rc.racer, body, position, quaternion_of(yaw))
        flying = (torch.rand(count, generator=g) < rc.flying_share * self.difficulty).to(dev)
        speed = (torch.rand(count, generator=g) * rc.start_speed).to(dev) * flying
        flight["velocity"] = normal * speed[:, None]
        lo, hi = rc.latency
        delay = torch.round((lo + (hi - lo) * torch.rand(count, generator=g) * self.ramp) * rc.hz).long().to(dev)
        rate_limit = (rc.rate_limit * (1 + rc.rate_spread * self.ramp * (2 * torch.rand(count, generator=g) - 1))).to(dev)
        hover_cmd = torch.cat([(body["mass"] * GRAVITY)[:, None], torch.zeros(count, 3, device=dev)], -1)
        state = {"course": course, "body": body, "flight": flight, "target": torch.zeros(count, dtype=torch.long, device=dev),
                 "distance": (first - position).norm(dim=-1), "steps": torch.zeros(count, dtype=torch.long, device=dev),
                 "passed": torch.zeros(count, dtype=torch.long, device=dev), "last_action": torch.zeros(count, 4, device=dev),
                 "pending": hover_cmd[:, None].expand(count, rc.max_delay + 1, 4).contiguous(), "delay": delay, "rate_limit": rate_limit,
                 "key": torch.full((count,), int(key), dtype=torch.long, device=dev)}
        zero = torch.zeros(count, device=dev)
        never = torch.zeros(count, dtype=torch.bool, device=dev)
        return state, TimeStep(self.observe(state), zero, never, never.clone())

    def step(self, state, action):
        rc = self.racing
        action = action.to(self.device).float().clamp(-1, 1)
        collective, rates = commanded(rc, state["body"], state["rate_limit"], action)
        pending, taken = delayed(state["pending"], torch.cat([collective[:, None], rates], -1), state["delay"])
        step_key = int(state["key"][0]) * 100003 + int(state["steps"].max()) + 1
        flight, path = flown(rc.racer, state["body"], state["flight"], taken[:, 0], taken[:, 1:], rc.hz, step_key)
        centre, facing = self._gate(state["course"], state["target"])
        crashed, passed, offset = struck(rc, path, centre, facing, state["course"]["obstacles"])
        # straying far past the gate's plane without passing it ends the episode too
        normal, _ = gate_axes(facing)
        beyond = ((flight["position"] - centre) * normal).sum(-1)
        missed = ~passed & (beyond > rc.miss_radius)
        after = (centre - flight["position"]).norm(dim=-1)
        dt = 1.0 / rc.hz
        reward = rc.progress_scale * (state["distance"] - after) \
            - rc.rate_cost * flight["angular_velocity"].norm(dim=-1) * dt * rc.hz / 60 \
            - rc.smoothness_cost * ((action - state["last_action"]) ** 2).sum(-1) \
            + rc.perception_scale * torch.exp(-rc.perception_sharpness * looking(rc, flight, centre) ** 4) \
            + passed * rc.gate_bonus * (1 - 0.5 * offset)
        target = state["target"] + passed.long()
        n_passed = state["passed"] + passed.long()
        finished = ~state["course"]["closed"] & (target >= state["course"]["count"])
        terminated = crashed | missed | finished
        reward = reward - rc.crash_penalty * (crashed | missed)
        steps = state["steps"] + 1
        truncated = (steps >= rc.episode_steps) & ~terminated
        new_centre, _ = self._gate(state["course"], target)
        new = {**state, "flight": flight, "target": target, "distance": (new_centre - flight["position"]).norm(dim=-1), "steps": steps,
               "passed": n_passed, "last_action": action, "pending": pending}
        return new, TimeStep(self.observe(new), reward, terminated, truncated)


# ------------------------------------------------------------------------------------------------ the race through a camera
class GateRace(Simulator, Branching):
    """``count`` drones racing ``racing``'s courses (``FlightEnv``) and seen through a ray-cast front camera: observations are the
    privileged ``views`` asked for plus ``image [N, H, W, 3]`` when a ``camera`` is given (motion-blurred between the poses at the
    shutter's opening - the step before - and its close)."""

    def __init__(self, count: int, racing: Racing = Racing(), views: Sequence[str] = ("state", "gates", "action"),
                 camera: Optional[Camera] = None, difficulty: float = 1.0, ramp: float = 1.0, device="cpu"):
        self.env = FlightEnv(racing, views, difficulty, ramp, device)
        self.count, self.action_size, self.camera, self.device = count, 4, camera, torch.device(device)
        self.state = None
        self.key = 0

    def _pose(self, flight) -> torch.Tensor:
        """A camera pose ``[N, 12]``: position, then the image's right, down and forward axes (the body's, tilted up)."""
        R = rotation(flight["orientation"])
        tilt = math.radians(self.env.racing.uptilt)
        fwd = R @ torch.tensor([math.cos(tilt), 0.0, math.sin(tilt)], device=self.device)
        up = R @ torch.tensor([-math.sin(tilt), 0.0, math.cos(tilt)], device=self.device)
        left = R @ torch.tensor([0.0, 1.0, 0.0], device=self.device)
        return torch.cat([flight["position"], -left, -up, fwd], -1)

    def scene(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """The boxes ``[N, 4 G, 10]`` of the course's gate frames (inactive gates shrunk to nothing, the gate headed for lit) and
        the pillars as cylinders ``[N, O, 7]``."""
        course = self.state["course"]
        N, G, _ = course["centres"].shape
        rc = self.env.racing
        boxes = gate_boxes(course["centres"], course["facing"], inner=rc.opening, bar=rc.frame, depth=rc.depth).reshape(N, G, 4, 10)
        idx = torch.arange(G, device=self.device)[None]
        live = idx < course["count"][:, None]
        boxes = torch.cat([boxes[..., :3], boxes[..., 3:6] * live[..., None, None], boxes[..., 6:]], -1)
        target = torch.where(course["closed"], self.state["target"] % course["count"], torch.minimum(self.state["target"], course["count"] - 1))
        lit = (idx == target[:, None])[..., None, None]
        colour = torch.where(lit, torch.tensor([1.0, 0.9, 0.2], device=self.device), boxes[..., 7:10])
        boxes = torch.cat([boxes[..., :7], colour], -1).reshape(N, G * 4, 10)
        obs = course["obstacles"]
        O = obs.shape[1]
        cyl = torch.stack([obs[..., 0], obs[..., 1], obs[..., 2], obs[..., 3], torch.full_like(obs[..., 0], 0.45), torch.full_like(obs[..., 0], 0.45),
                           torch.full_like(obs[..., 0], 0.5)], -1)
        return boxes, cyl

    def _observe(self, observation, before) -> Dict[str, torch.Tensor]:
        out = dict(observation)
        if self.camera is not None:
            boxes, cyl = self.scene()
            poses = torch.stack([self._pose(before), self._pose(self.state["flight"])], 1)
            out["image"] = render(poses, boxes, cyl, self.camera)
        return out

    def reset(self, seed: int):
        self.key = int(seed) + 1
        self.state, ts = self.env.reset(int(seed), self.count)
        self._obs = self._observe(ts.observation, self.state["flight"])
        return self._obs

    def step(self, action):
        before = self.state["flight"]
        self.state, ts = self.env.step(self.state, action)
        self._obs = self._observe(ts.observation, before)
        return self._obs, ts.reward, ts.terminated, ts.truncated

    def restart(self, mask):
        fresh, first = self.env.reset(self.key, self.count)
        self.key += 1
        mask = mask.to(self.device)
        self.state = chosen(mask, fresh, self.state)
        self._obs = chosen(mask, self._observe(first.observation, self.state["flight"]), self._obs)
        return self._obs

    def snapshot(self):
        clone = lambda x: x.clone()
        return tree_map(clone, self.state), tree_map(clone, self._obs), self.key

    def restore(self, snapshot):
        self.state, self._obs, self.key = snapshot
