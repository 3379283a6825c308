"""Environments as two functions over a state tree, and the one loop over them.

An ``Env`` here is batched from the start (torch tensors lead with the environment axis): ``reset(key, count) -> (state,
TimeStep)`` and ``step(state, action) -> (state, TimeStep)``, both functions of their arguments alone - the state is a tree
(dict / dataclass / tuple) of tensors the caller holds.  A simulator has this shape and so has a learned world model, whose
state is its latent and whose step is the learned dynamics; acting in a simulator and imagining in a world model are the same
``env_rollout``.

An episode that ends restarts in place: the transition that ended it is recorded first, then the ended environments take a
fresh state (``chosen``), as auto-reset wrappers do.  ``TimeLimit`` cuts episodes after a number of steps and repeats actions;
``Driven`` presents the whole step (observation, reward, first / last / terminal flags) as the observation a world-model
learner records.

Reference: src/dew/rl/env.py (``TimeStep``, ``Env``, ``chosen``, ``TimeLimit``, ``Batched``, ``Transition``, ``Carry``, ``start``,
``env_step``, ``env_rollout``, ``Driven``).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple

import torch

Tree = Any


def tree_map(fn: Callable, *trees: Tree) -> Tree:
    t = trees[0]
    if isinstance(t, torch.Tensor):
        return fn(*trees)
    if dataclasses.is_dataclass(t) and not isinstance(t, type):
        return type(t)(**{f.name: tree_map(fn, *(getattr(x, f.name) for x in trees)) for f in dataclasses.fields(t)})
    if isinstance(t, Mapping):
        return type(t)((k, tree_map(fn, *(x[k] for x in trees))) for k in t)
    if isinstance(t, (tuple, list)):
        return type(t)(tree_map(fn, *xs) for xs in zip(*trees))
    return t                                                             # a static leaf (an int, None, a string)


def chosen(mask: torch.Tensor, new: Tree, old: Tree) -> Tree:
    """``new`` where ``mask [N]`` holds, ``old`` elsewhere, leaf by leaf along the leading axis."""
    def pick(a, b):
        m = mask.reshape(mask.shape + (1,) * (a.dim() - mask.dim()))
        return torch.where(m, a, b)
    return tree_map(pick, new, old)


def views(observation) -> Dict[str, torch.Tensor]:
    return dict(observation) if isinstance(observation, Mapping) else {"observation": observation}


def view(observation, name: Optional[str] = None) -> torch.Tensor:
    return observation if name is None else observation[name]


@dataclass
class TimeStep:
    observation: Tree
    reward: torch.Tensor            # [N], zero at a reset
    terminated: torch.Tensor        # [N] bool: ended in a terminal state, whose value is zero
    truncated: torch.Tensor         # [N] bool: cut (a time limit), the state's value stands

    @property
    def done(self) -> torch.Tensor:
        return self.terminated | self.truncated


class Env:
    action_size: int = 0

    def reset(self, key: int, count: int) -> Tuple[Tree, TimeStep]:
        raise NotImplementedError

    def step(self, state: Tree, action: torch.Tensor) -> Tuple[Tree, TimeStep]:
        raise NotImplementedError


class TimeLimit(Env):
    """``env`` whose episodes are cut after ``episode_length`` steps, each step repeating its action ``action_repeat`` times and
    summing the rewards (an environment that ends inside the repeats stops earning)."""

    def __init__(self, env: Env, episode_length: int, action_repeat: int = 1):
        self.env, self.episode_length, self.action_repeat = env, episode_length, action_repeat
        self.action_size = env.action_size

    def reset(self, key, count):
        state, ts = self.env.reset(key, count)
        return {"inner": state, "steps": torch.zeros(count, dtype=torch.long, device=ts.reward.device)}, ts

    def step(self, state, action):
        inner, steps = state["inner"], state["steps"]
        live = torch.ones_like(steps, dtype=torch.bool)
        total = term = ended = obs = None
        for r in range(self.action_repeat):
            nxt, ts = self.env.step(inner, action)
            inner = nxt if r == 0 else chosen(live, nxt, inner)
            obs = ts.observation if r == 0 else chosen(live, ts.observation, obs)
            total = ts.reward * live if r == 0 else total + ts.reward * live
            term = (ts.terminated & live) if r == 0 else term | (ts.terminated & live)
            ended = (ts.done & live) if r == 0 else ended | (ts.done & live)
            live = ~ended
        steps = steps + 1
        cut = (steps >= self.episode_length) & ~term
        return {"inner": inner, "steps": steps}, TimeStep(obs, total, term, cut | (ended & ~term))


@dataclass
class Transition:
    """One step of a rollout, leading with the environment axis: the observation acted on, the action taken, what the policy
    reported beside it (log-probability, value ...), and the step that answered."""
    observation: Tree
    action: torch.Tensor
    extras: Dict[str, torch.Tensor]
    step: TimeStep


@dataclass
class Carry:
    state: Tree
    observation: Tree
    key: int
    memory: Tree = None
    episodes: int = 0


Policy = Callable[[Any, Tree, Tree, int], Tuple[torch.Tensor, Dict[str, torch.Tensor], Tree]]
"""``policy(params, observation, memory, key) -> (action, extras, memory)``."""


def start(env: Env, key: int, count: int, memory: Tree = None) -> Carry:
    state, ts = env.reset(key, count)
    return Carry(state, ts.observation, key + 1, memory)


def env_step(env: Env, policy: Policy, params, carry: Carry, reset: bool = True, reset_memory: Optional[Callable[[Tree, torch.Tensor], Tree]] = None
             ) -> Tuple[Carry, Transition]:
    action, extras, memory = policy(params, carry.observation, carry.memory, carry.key)
    state, ts = env.step(carry.state, action)
    tr = Transition(carry.observation, action, extras, ts)
    obs = ts.observation
    key = carry.key + 1
    if reset:
        done = ts.done
        if bool(done.any()):
            fresh, first = env.reset(key, done.shape[0])
            key += 1
            state = chosen(done, fresh, state)
            obs = chosen(done, first.observation, obs)
            if reset_memory is not None:
                memory = reset_memory(memory, done)
    return Carry(state, obs, key, memory, carry.episodes + int(ts.done.sum())), tr


def stack_transitions(steps: List[Transition]) -> Transition:
    cat = lambda *xs: torch.stack(xs)
    return Transition(tree_map(cat, *[s.observation for s in steps]), torch.stack([s.action for s in steps]),
                      {k: torch.stack([s.extras[k] for s in steps]) for k in steps[0].extras},
                      TimeStep(tree_map(cat, *[s.step.observation for s in steps]), torch.stack([s.step.reward for s in steps]),
                               torch.stack([s.step.terminated for s in steps]), torch.stack([s.step.truncated for s in steps])))


def env_rollout(env: Env, policy: Policy, params, carry: Carry, steps: int, reset: bool = True, reset_memory=None) -> Tuple[Carry, Transition]:
    """``steps`` steps of ``policy`` in ``env`` from ``carry``: the carry after them and every step's ``Transition``, leading with
    the step axis ``[steps, N, ...]``."""
    out = []
    for _ in range(steps):
        carry, tr = env_step(env, policy, params, carry, reset, reset_memory)
        out.append(tr)
    return carry, stack_transitions(out)


class Driven(Env):
    """``env`` stepped as an agent's driver steps it: its observation is the whole step a world-model learner records - the
    observation's views, the ``reward`` that came with them, and whether the step is its episode's ``first``, its ``last`` or
    ``terminal``.  An ended episode restarts on the next step (that step's action is ignored and its observation is ``first``)."""

    def __init__(self, env: Env):
        self.env, self.action_size = env, env.action_size

    @staticmethod
    def driven_step(ts: TimeStep, first: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {**views(ts.observation), "reward": ts.reward, "first": first, "last": ts.done, "terminal": ts.terminated}

    def reset(self, key, count):
        state, ts = self.env.reset(key, count)
        first = torch.ones(count, dtype=torch.bool, device=ts.reward.device)
        obs = self.driven_step(ts, first)
        return {"inner": state, "ended": torch.zeros_like(first), "key": key + 1}, TimeStep(obs, ts.reward, ts.terminated, ts.truncated)

    def step(self, state, action):
        ended = state["ended"]
        nxt, ts = self.env.step(state["inner"], action)
        key = state["key"]
        if bool(ended.any()):
            fresh, first = self.env.reset(key, ended.shape[0])
            key += 1
            nxt = chosen(ended, fresh, nxt)
            ts = TimeStep(chosen(ended, first.observation, ts.observation), torch.where(ended, torch.zeros_like(ts.reward), ts.reward),
                          ts.terminated & ~ended, ts.truncated & ~ended)
        obs = self.driven_step(ts, ended)
        # the wrapper itself never ends: the flags live in the observation
        never = torch.zeros_like(ended)
        return {"inner": nxt, "ended": ts.done, "key": key}, TimeStep(obs, ts.reward, never, never)
