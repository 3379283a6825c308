"""Reinforcement learning on plain tensors and plain functions: its math, its environments, their physics and camera, replays and
simulators.

The math is ``advantage`` (rewards -> advantages), ``surrogate`` (log-probabilities and advantages -> loss terms) and
``distributions`` (DreamerV3's transforms and categoricals); none of them knows a model, an objective or a batch dict.  An
environment is an ``env.Env`` (reset / step over a state tree, ``env_rollout`` the one loop that acts in it); ``simulator`` is the
boundary for an engine stepped from the host; ``replay`` keeps steps on the device; ``evaluation`` scores a policy by its first
episodes; ``aggregation`` labels a student's steps with a privileged teacher's actions (DAgger); ``sandbox`` runs programs and
tool sessions in bounded subprocesses for verifiable rewards.  The drone race is ``quadrotor`` (a racing quadrotor's physics,
randomised per episode), ``flight`` (courses, gates, collisions, the reward; ``FlightEnv`` and the camera-seen ``GateRace``) and
``camera`` (a CUDA ray caster with a torch restatement).

Reference: src/dew/rl/ (advantage, surrogate, distributions, env, simulator, replay, evaluation, aggregation, sandbox, quadrotor,
flight, hyperlux).
"""
from . import advantage, aggregation, distributions, env, evaluation, sandbox, simulator, surrogate
from .advantage import (discounted_returns, dr_grpo_advantage, gae, gae_advantages, generalized_advantages, group_advantage, lambda_returns,
                        masked_mean, masked_whiten, rloo_advantage)
from .camera import Camera, fisheye_map, fisheyed, gate_boxes, look_at, render, render_reference
from .env import Carry, Driven, Env, TimeLimit, TimeStep, Transition, env_rollout, env_step, start
from .evaluation import episodes, first_episode_rows, first_episodes
from .flight import FlightEnv, GateRace, Racing
from .quadrotor import Quadrotor, QuadrotorState, Racer, drawn_body, flown, hovering
from .replay import Replay, ReplayBuffer
from .sandbox import MathReward, Outcome, ProcessRunner, Program, ProgramReward, SandboxFleet, SandboxLimits, SubprocessEnvironment, Verdict, outputs_match
from .simulator import DrivenSimulator, EnvSimulator, Simulator, simulator_rollout, simulator_start

__all__ = [n for n in dir() if not n.startswith("_")]
