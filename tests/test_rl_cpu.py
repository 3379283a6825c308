"""Quadrotor dynamics, the gate race, advantages, replay, and the camera's CPU restatement."""
import math

import torch

from dew_b200.rl import (Camera, GateRace, Quadrotor, Replay, discounted_returns, fisheye_map, fisheyed, gate_boxes,
                         generalized_advantages, look_at, render_reference)


def test_quadrotor_hovers_and_falls():
    m = Quadrotor()
    s = m.reset(2)
    hover = torch.full((2, 4), 2 * (m.mass * m.g / 4) / m.thrust_max - 1)
    for _ in range(100):
        s = m.step(s, hover)
    assert (s.position[:, 2] - 1.0).abs().max() < 1e-3 and (s.quaternion.norm(dim=-1) - 1).abs().max() < 1e-6
    s2 = m.reset(1)
    for _ in range(50):
        s2 = m.step(s2, -torch.ones(1, 4))
    assert float(s2.position[0, 2]) < 0.5 * 1.0 + 0.5


def test_gae_matches_closed_form_and_replay_samples():
    r = torch.ones(4, 1); v = torch.zeros(4, 1); d = torch.zeros(4, 1, dtype=torch.bool)
    adv, ret = generalized_advantages(r, v, d, gamma=0.5, lam=1.0)
    assert torch.allclose(ret[:, 0], torch.tensor([1.875, 1.75, 1.5, 1.0]))
    assert torch.allclose(discounted_returns(r, d, 0.5)[:, 0], torch.tensor([1.875, 1.75, 1.5, 1.0]))
    rp = Replay(8)
    rp.add({"x": torch.arange(12.0)[:, None]})
    assert rp.size == 8 and set(rp.store["x"][:, 0].tolist()) == set(range(4, 12))
    assert rp.sample(5, torch.Generator().manual_seed(0))["x"].shape == (5, 1)


def test_camera_sees_gate_ground_and_sky():
    cam = Camera(size=(48, 64), fov=90.0, fisheye=False, samples=1, fog=0.0)
    pos = torch.tensor([[0.0, 0.0, 1.5]])
    cams = look_at(pos, torch.tensor([[5.0, 0.0, 1.5]]))[:, None]
    boxes = gate_boxes(torch.tensor([[5.0, 0.0, 1.5]]), torch.tensor([0.0]), color=(1.0, 0.0, 0.0)).reshape(1, 4, 10)
    cyl = torch.tensor([[[3.0, 2.0, 0.2, 3.0, 0.0, 0.0, 1.0]]])
    img = render_reference(cams, boxes, cyl, cam)
    assert img.shape == (1, 48, 64, 3)
    centre, top, bottom = img[0, 22, 32], img[0, 1, 32], img[0, 46, 32]
    assert centre[2] > centre[0]                       # through the opening: sky
    assert bottom[1] > 0.2 and abs(float(bottom[0] - 0.9 * bottom[1])) < 1e-5       # ground checker tint
    red = (img[0, ..., 0] > 0.3) & (img[0, ..., 1] < 0.05)
    assert red.sum() > 20                              # the gate's bars
    blue = (img[0, ..., 2] > 0.3) & (img[0, ..., 0] < 0.05) & (img[0, ..., 1] < 0.05)
    assert blue.sum() > 5                              # the pillar, to the left of the gate (world +y is image left)
    assert blue.nonzero()[:, 1].float().mean() < 32


def test_fisheye_direct_cast_matches_resampled_pinhole():
    """Casting the fisheye directly and resampling a large pinhole agree where the pinhole holds the direction."""
    pos = torch.tensor([[0.0, 0.0, 1.2]])
    cams = look_at(pos, torch.tensor([[4.0, 0.5, 1.4]]))[:, None]
    boxes = gate_boxes(torch.tensor([[4.0, 0.0, 1.5]]), torch.tensor([0.2])).reshape(1, 4, 10)
    cyl = torch.zeros(1, 0, 7)
    fish = render_reference(cams, boxes, cyl, Camera(size=(32, 32), fov=100.0, fisheye=True, samples=1))
    pin = render_reference(cams, boxes, cyl, Camera(size=(256, 256), fov=100.0, fisheye=False, samples=1))
    corners, weights, held = fisheye_map(32, 256, 100.0)
    resampled = fisheyed(pin, corners, weights)
    close = ((fish - resampled).abs().max(-1).values < 0.08) | ~held[None]
    assert close.float().mean() > 0.93                 # edges of bars differ by the resampling blur only


def test_gate_race_steps_with_images():
    env = GateRace(3, camera=Camera(size=(24, 24)), views=("state", "gates"))
    obs = env.reset(1)
    assert obs["state"].shape == (3, 13) and obs["gates"].shape == (3, 24) and obs["image"].shape == (3, 24, 24, 3)
    total = torch.zeros(3)
    for _ in range(20):
        obs, r, terminated, truncated = env.step(torch.zeros(3, 4))
        total += r
    assert torch.isfinite(total).all() and torch.isfinite(obs["image"]).all() and not bool(truncated.any())
    # the gate headed for is in view at the start: its lit frame colours some pixels
    first = GateRace(2, camera=Camera(size=(48, 48), fov=110.0, fog=0.0), difficulty=0.0, ramp=0.0).reset(3)["image"]
    lit = (first[..., 0] > first[..., 1]) & (first[..., 1] > 2 * first[..., 2]) & (first[..., 0] > 0.2)
    assert int(lit[0].sum()) > 30
    # a branch steps the race and leaves it as it was
    before = env.state["flight"]["position"].clone()
    with env.branch():
        env.step(torch.ones(3, 4))
    assert torch.equal(env.state["flight"]["position"], before)
    restarted = env.restart(torch.tensor([True, False, False]))
    assert int(env.state["steps"][0]) == 0 and int(env.state["steps"][1]) == 20 and restarted["state"].shape == (3, 13)


def test_dreamer_actor_critic_improves_imagined_return():
    """In a known world (reward = -|z|^2, dynamics z' = z + 0.3 a) the actor learns to drive the state to the origin."""
    import torch
    from dew_b200.objectives.base import Step
    from dew_b200.objectives.consistency import DreamerObjective, lambda_returns

    class World(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.pi = torch.nn.Sequential(torch.nn.Linear(2, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
            self.v = torch.nn.Sequential(torch.nn.Linear(2, 32), torch.nn.Tanh(), torch.nn.Linear(32, 1))

        def encode(self, obs): return obs
        def dynamics(self, z, a): return z + 0.3 * a
        def reward(self, z, a): return -(z ** 2).sum(-1)
        def done(self, z): return torch.full((z.shape[0],), -10.0)
        def actor(self, z): return self.pi(z).chunk(2, -1)
        def critic(self, z): return self.v(z).squeeze(-1)

    torch.manual_seed(0)
    w = World()
    obj = DreamerObjective(w, horizon=8)
    opt = torch.optim.Adam(w.parameters(), lr=3e-3)
    returns = []
    for it in range(120):
        obs = torch.randn(64, 2, generator=torch.Generator().manual_seed(it))
        stats, aux = obj.loss(None, {"observation": obs}, Step(train=True, key=it))
        opt.zero_grad(); stats.value().backward(); opt.step()
        returns.append(float(aux.metrics["imagined_return"].value()))
    assert sum(returns[-10:]) / 10 > sum(returns[:10]) / 10 + 0.5
    # lambda-returns: with lam = 1 they are the discounted sums plus the bootstrap
    r, c, v = torch.ones(3, 1), torch.full((3, 1), 0.5), torch.zeros(4, 1)
    assert torch.allclose(lambda_returns(r, v, c, 1.0)[:, 0], torch.tensor([1.75, 1.5, 1.0]))
