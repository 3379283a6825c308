"""A simulator stepped from the host as an environment: the boundary any external engine (a CUDA, Warp, C++ or game engine)
plugs into.

Such an engine keeps its own state, so it is not an ``Env`` (functions of a state tree); it is ``Stepped``: ``reset(seed)``
starts every episode and ``step(action)`` advances every environment by its row of the ``[count, action_size]`` action.  A
``Simulator`` restarts none by itself: ``restart(mask)`` starts a new episode where ``mask`` selects, so the driver decides when an
ended episode restarts - ``simulator_rollout`` restarts it at once and records what ``env_rollout`` records.  Arrays cross the
boundary by DLPack (``taken``): without a copy where both sides hold them on one device, then cloned, since an engine may write
its next step into the same memory.

Reference: src/dew/rl/simulator.py (``Stepped``, ``Simulator``, ``Branching``, ``taken``, ``received``, ``simulator_start``,
``simulator_rollout``, ``DrivenSimulator``, ``rollout_start``).
"""
from __future__ import annotations

import contextlib
from typing import Any, Dict, Mapping, Optional, Tuple

import numpy as np
import torch

from .env import Carry, Driven, Env, TimeStep, Transition, chosen, stack_transitions, start, tree_map, views


class Stepped:
    count: int = 0
    action_size: int = 0

    def reset(self, seed: int) -> Any:
        raise NotImplementedError

    def step(self, action: torch.Tensor) -> Tuple[Any, Any, Any, Any]:
        """-> (observation, reward [count], terminated [count], truncated [count])"""
        raise NotImplementedError


class Simulator(Stepped):
    def restart(self, mask: torch.Tensor) -> Any:
        """Start a new episode in each environment ``mask [count]`` selects; answer every environment's observation."""
        raise NotImplementedError


class Branching:
    """A simulator a side branch (an evaluation, a cooldown) may step and then leave as the run left it."""

    def snapshot(self) -> Any:
        raise NotImplementedError

    def restore(self, snapshot: Any) -> None:
        raise NotImplementedError

    @contextlib.contextmanager
    def branch(self):
        held = self.snapshot()
        try:
            yield self
        finally:
            self.restore(held)


def branched(simulator):
    if not isinstance(simulator, Branching):
        raise TypeError(f"{type(simulator).__name__} cannot be stepped in a branch: it has no snapshot / restore")
    return simulator.branch()


def taken(array, device=None) -> torch.Tensor:
    """A simulator's array as a tensor of our own: another framework's through DLPack, a NumPy array by copy."""
    if isinstance(array, torch.Tensor):
        out = array.clone()
    elif isinstance(array, np.ndarray):
        out = torch.from_numpy(np.array(array, copy=True))
    elif hasattr(array, "__dlpack__"):
        out = torch.from_dlpack(array).clone()
    else:
        out = torch.as_tensor(array)
    return out if device is None else out.to(device)


def received(tree, device=None):
    if isinstance(tree, Mapping):
        return {k: received(v, device) for k, v in tree.items()}
    if isinstance(tree, (tuple, list)):
        return type(tree)(received(v, device) for v in tree)
    return taken(tree, device)


def simulator_start(simulator: Stepped, key: int, memory=None, device=None) -> Carry:
    return Carry(None, received(simulator.reset(int(key)), device), key + 1, memory)


def simulator_rollout(simulator: Simulator, policy, params, carry: Carry, steps: int, reset: bool = True, reset_memory=None, device=None
                      ) -> Tuple[Carry, Transition]:
    out = []
    for _ in range(steps):
        action, extras, memory = policy(params, carry.observation, carry.memory, carry.key)
        obs, reward, terminated, truncated = simulator.step(action)
        ts = TimeStep(received(obs, device), taken(reward, device).float(), taken(terminated, device).bool(), taken(truncated, device).bool())
        out.append(Transition(carry.observation, action, extras, ts))
        nxt = ts.observation
        done = ts.done
        if reset and bool(done.any()):
            nxt = received(simulator.restart(done), device)
            if reset_memory is not None:
                memory = reset_memory(memory, done)
        carry = Carry(None, nxt, carry.key + 1, memory, carry.episodes + int(done.sum()))
    return carry, stack_transitions(out)


class EnvSimulator(Simulator, Branching):
    """An ``Env`` held as a simulator (its state kept inside): what a test or a driver written against ``Simulator`` steps."""

    def __init__(self, env: Env, count: int):
        self.env, self.count, self.action_size = env, count, env.action_size
        self.state, self.key = None, 0

    def reset(self, seed):
        self.key = int(seed) + 1
        self.state, ts = self.env.reset(int(seed), self.count)
        self._obs = ts.observation
        return ts.observation

    def step(self, action):
        self.state, ts = self.env.step(self.state, action)
        self._obs = ts.observation
        return ts.observation, ts.reward, ts.terminated, ts.truncated

    def restart(self, mask):
        fresh, first = self.env.reset(self.key, self.count)
        self.key += 1
        self.state = chosen(mask, fresh, self.state)
        self._obs = chosen(mask, first.observation, self._obs)
        return self._obs

    def snapshot(self):
        clone = lambda x: x.clone()
        return tree_map(clone, self.state), tree_map(clone, self._obs), self.key

    def restore(self, snapshot):
        self.state, self._obs, self.key = snapshot


class DrivenSimulator(Stepped):
    """``simulator`` driven as ``Driven`` drives an ``Env``: the observation is the whole step (views, reward, first / last /
    terminal); an ended episode restarts on the next step, whose action is ignored."""

    def __init__(self, simulator: Simulator, device=None):
        self.simulator, self.count, self.action_size, self.device = simulator, simulator.count, simulator.action_size, device
        self.ended = None

    def reset(self, seed):
        obs = received(self.simulator.reset(seed), self.device)
        n = self.count
        dev = next(iter(views(obs).values())).device
        self.ended = torch.zeros(n, dtype=torch.bool, device=dev)
        zero = torch.zeros(n, device=dev)
        self._last = obs
        return {**views(obs), "reward": zero, "first": ~self.ended, "last": self.ended.clone(), "terminal": self.ended.clone()}

    def step(self, action):
        ended = self.ended
        obs, reward, terminated, truncated = self.simulator.step(action)
        obs, reward = received(obs, self.device), taken(reward, self.device).float()
        terminated, truncated = taken(terminated, self.device).bool(), taken(truncated, self.device).bool()
        if bool(ended.any()):
            # the environments that had ended restart now; what their ignored action did is discarded
            obs = received(self.simulator.restart(ended), self.device)
            reward = torch.where(ended, torch.zeros_like(reward), reward)
            terminated, truncated = terminated & ~ended, truncated & ~ended
        done = terminated | truncated
        self.ended = done
        never = torch.zeros_like(done)
        return {**views(obs), "reward": reward, "first": ended, "last": done, "terminal": terminated}, reward, never, never


def rollout_start(env, key: int, count: Optional[int] = None, memory=None) -> Carry:
    if isinstance(env, Env):
        return start(env, key, count, memory)
    return simulator_start(env, key, memory)
