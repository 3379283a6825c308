"""PPO for continuous control: GAE that tells termination from truncation, and a policy that learns to drive a point mass to the origin."""
import math

import torch

from dew_b200.objectives.rl.control import ActorCritic, ControlPPO, RunningMoments, episode_gae
from dew_b200.rl.env import Env, TimeLimit, TimeStep


class PointMass(Env):
    """A point on a line pushed by the action; reward is minus the distance to the origin; leaving [-3, 3] is terminal."""
    action_size, observation_size = 1, 2

    def reset(self, key, count):
        g = torch.Generator().manual_seed(int(key))
        state = {"x": torch.rand(count, generator=g) * 2 - 1, "v": torch.zeros(count)}
        return state, TimeStep(torch.stack([state["x"], state["v"]], -1), torch.zeros(count), torch.zeros(count, dtype=torch.bool), torch.zeros(count, dtype=torch.bool))

    def step(self, state, action):
        v = 0.8 * state["v"] + 0.2 * action[:, 0].clamp(-1, 1)
        x = state["x"] + 0.3 * v
        out = x.abs() > 3
        return {"x": x, "v": v}, TimeStep(torch.stack([x, v], -1), -x.abs() - 5.0 * out.float(), out, torch.zeros_like(out))


def test_episode_gae_separates_termination_from_truncation():
    r = torch.tensor([[1.0], [1.0], [1.0]])
    v = torch.tensor([[0.5], [0.5], [0.5]])
    nv = torch.tensor([[0.5], [0.5], [2.0]])
    none = torch.zeros(3, 1, dtype=torch.bool)
    last = torch.tensor([[False], [False], [True]])
    adv_trunc, _ = episode_gae(r, v, nv, none, last, gamma=0.9, lam=1.0)
    adv_term, _ = episode_gae(r, v, nv, last, last, gamma=0.9, lam=1.0)
    assert adv_trunc[2, 0] == (1 + 0.9 * 2.0 - 0.5) and adv_term[2, 0] == (1 - 0.5)
    assert math.isclose(float(adv_term[0, 0]), 1 + 0.9 + 0.81 - 0.5, rel_tol=1e-6)       # lam 1: the discounted return minus the value
    mid = torch.tensor([[False], [True], [False]])                                        # an episode ends mid-rollout: nothing flows across it
    adv, _ = episode_gae(r, v, nv, mid, mid, gamma=0.9, lam=1.0)
    assert adv[1, 0] == 0.5 and math.isclose(float(adv[0, 0]), 1 + 0.9 * 1 - 0.5, rel_tol=1e-6)
    m = RunningMoments(2)
    x = torch.randn(500, 2) * torch.tensor([2.0, 0.5]) + torch.tensor([1.0, -3.0])
    m.update(x[:200]), m.update(x[200:])
    assert torch.allclose(m.mean, x.mean(0), atol=1e-3) and torch.allclose(m.var, x.var(0, unbiased=False), atol=1e-2)


def test_ppo_learns_to_hold_a_point_mass_at_the_origin():
    torch.manual_seed(0)
    env = TimeLimit(PointMass(), episode_length=40)
    model = ActorCritic(2, 1, hidden=(32, 32))
    ppo = ControlPPO(env, model, envs=32, steps=40, epochs=4, minibatches=4, learning_rate=3e-3, gamma=0.95, seed=1)
    history = ppo.train(30)
    first = [h["episode_return"] for h in history[:3] if not math.isnan(h["episode_return"])]
    last = [h["episode_return"] for h in history[-3:]]
    assert sum(last) / len(last) > sum(first) / len(first) + 5.0, (first, last)
    assert sum(last) / len(last) > -8.0, last                     # a still policy averages about -20 from a uniform start
    action, _ = model.act(torch.tensor([[1.0, 0.0], [-1.0, 0.0]]), greedy=True)
    assert float(action[0]) < 0 < float(action[1])                 # push towards the origin
    assert 0.0 <= history[-1]["clip_fraction"] <= 1.0 and history[-1]["entropy"] == history[-1]["entropy"]
