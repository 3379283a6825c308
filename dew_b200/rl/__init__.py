"""Reinforcement-learning environments and helpers: quadrotor dynamics, the gate-race task and its camera (a CUDA ray
caster), advantages and a replay buffer.  Reference: src/dew/rl/{quadrotor,flight,simulator,hyperlux,advantage,replay}.py."""
from .advantage import discounted_returns, generalized_advantages
from .camera import Camera, fisheye_map, fisheyed, gate_boxes, look_at, render, render_reference
from .quadrotor import Quadrotor, QuadrotorState
from .flight import GateRace
from .replay import Replay

__all__ = ["Camera", "GateRace", "Quadrotor", "QuadrotorState", "Replay", "discounted_returns", "fisheye_map", "fisheyed",
           "gate_boxes", "generalized_advantages", "look_at", "render", "render_reference"]
