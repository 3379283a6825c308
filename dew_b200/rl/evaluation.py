"""A policy scored by the episodes it plays rather than by records it reads.

``episodes(policy, env, steps)`` returns a scorer: called with the policy's parameters and a key, it plays fresh environments
``steps`` steps without restarting and returns means over each environment's *first* episode - the undiscounted ``return``, the
``steps`` it lasted, the share ``terminated`` (not cut), and for each named observation view its value at the episode's last
step - so a score is one an episode earns once, however long the rollout runs past it.

Reference: src/dew/rl/evaluation.py (``first_episodes``, ``first_episode_rows``, ``flights``, ``episodes``).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence

import torch

from .env import Env, Transition, env_rollout, start, views
from .simulator import Simulator, simulator_rollout, simulator_start


def first_episodes(done: torch.Tensor) -> torch.Tensor:
    """``done [T, N]`` -> ``[T, N]`` bool: the steps of each environment's first episode, the step that ended it included."""
    ended_before = torch.cat([torch.zeros_like(done[:1]), done[:-1]]).long().cumsum(0) > 0
    return ~ended_before


def first_episode_rows(steps: Transition, names: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    ts = steps.step
    inside = first_episodes(ts.done)
    last = (inside.long().sum(0) - 1).clamp_min(0)                                       # index of each first episode's last step
    n = torch.arange(last.shape[0], device=last.device)
    rows = {"return": (ts.reward * inside).sum(0), "steps": inside.sum(0).float(), "terminated": ts.terminated[last, n].float(),
            "finished": ts.done[last, n].float(), "last_reward": ts.reward[last, n]}
    obs = views(ts.observation)
    for name in names:
        rows[name] = obs[name][last, n].float()
    return rows


def flights(policy, env, steps: int, count: Optional[int] = None) -> Callable:
    def fly(params, key: int) -> Transition:
        with torch.no_grad():
            if isinstance(env, Env):
                _, tr = env_rollout(env, policy, params, start(env, key, count), steps, reset=False)
            else:
                _, tr = simulator_rollout(env, policy, params, simulator_start(env, key), steps, reset=False)
        return tr
    return fly


def episodes(policy, env, steps: int, count: Optional[int] = None, names: Sequence[str] = ()) -> Callable:
    fly = flights(policy, env, steps, count)

    def score(params, key: int) -> Dict[str, float]:
        rows = first_episode_rows(fly(params, key), names)
        return {k: float(v.float().mean()) for k, v in rows.items()}
    return score
