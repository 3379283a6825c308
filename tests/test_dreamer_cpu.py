"""DreamerV3 on a small control task: the world model learns to predict, imagination trains the actor, the policy acts in the loop."""
import torch

import dew_b200 as dew
from dew_b200.objectives.rl.dreamer import DreamerModel, DreamerPolicy, DreamerRollout, DreamerV3
from dew_b200.rl.env import Env, TimeLimit, TimeStep


class Reach(Env):
    """A point on [-1, 1] and a target: the action moves the point, the reward is minus the distance left."""
    action_size = 1

    def _obs(self, x, target):
        return {"observation": torch.stack([x, target], -1)}

    def reset(self, key, count):
        g = torch.Generator().manual_seed(int(key))
        x, target = torch.rand(count, generator=g) * 2 - 1, torch.rand(count, generator=g) * 2 - 1
        never = torch.zeros(count, dtype=torch.bool)
        return {"x": x, "target": target}, TimeStep(self._obs(x, target), torch.zeros(count), never, never.clone())

    def step(self, state, action):
        x = (state["x"] + 0.25 * action[:, 0].clamp(-1, 1)).clamp(-1, 1)
        reward = -(x - state["target"]).abs()
        never = torch.zeros_like(x, dtype=torch.bool)
        return {"x": x, "target": state["target"]}, TimeStep(self._obs(x, state["target"]), reward, never, never.clone())


def test_dreamer_learns_a_world_model_and_improves_its_policy():
    torch.manual_seed(0)
    env = TimeLimit(Reach(), episode_length=16)
    model = DreamerModel(observation=2, action=1, deter=64, stoch=4, classes=8, hidden=64, bins=63)
    objective = DreamerV3(model, horizon=8, gamma=0.95, entropy=1e-3)
    policy = DreamerPolicy(model)
    rollout = DreamerRollout(env, count=16, capacity=256)
    first = rollout.collect(policy, 64, key=0)
    batch = rollout.sample(8, 16, torch.Generator().manual_seed(0))
    assert batch["observation"].shape == (8, 16, 2) and batch["action"].shape == (8, 16, 1) and batch["first"].dtype == torch.bool
    # a window's stored action is the one that led to its step: the point moved by it (except across an episode's start)
    moved = batch["observation"][:, 1:, 0] - batch["observation"][:, :-1, 0]
    inside = ~batch["first"][:, 1:] & (batch["observation"][:, 1:, 0].abs() < 0.999)
    assert torch.allclose(moved[inside], 0.25 * batch["action"][:, 1:, 0][inside], atol=1e-5)
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=2e-3, weight_decay=0.0, clip_grads=100.0), tracker=(t := dew.MemoryTracker()))
    state, rewards = None, [first["reward"]]
    g = torch.Generator().manual_seed(1)
    for round_ in range(48):
        batches = [rollout.sample(16, 16, g) for _ in range(10)]
        state = trainer.fit(batches, state=state, steps=10 * (round_ + 1), log_every=10)
        rewards.append(rollout.collect(policy, 32, key=round_ + 1)["reward"])
    rows = t.rows
    assert rows[-1]["reward_loss"] < 0.6 * rows[0]["reward_loss"] and rows[-1]["recon"] < 0.5 * rows[0]["recon"]
    assert all(torch.isfinite(torch.tensor(r["loss"])) for r in rows) and rows[-1]["return_scale"] >= 1.0
    # the slow critic follows the critic, and took no optimizer step of its own
    gap = sum(float((a - b).abs().sum()) for a, b in zip(model.slow_critic.parameters(), model.critic.parameters()))
    assert 0 < gap and all(not p.requires_grad for p in model.slow_critic.parameters())
    # acting improved: the last rounds' mean reward beats the untrained policy's
    assert sum(rewards[-3:]) / 3 > rewards[0] + 0.2, rewards
    # a greedy policy from a filtered state is deterministic
    greedy = DreamerPolicy(model, greedy=True)
    obs = {"observation": torch.tensor([[0.5, -0.5]]), "first": torch.tensor([True])}
    a1, _, mem = greedy(None, obs, None, 0)
    a2, _, _ = greedy(None, obs, None, 5)
    assert torch.equal(a1, a2) and a1.shape == (1, 1) and len(mem) == 3
