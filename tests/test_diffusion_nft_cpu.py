"""DiffusionNFT: the loss's gradient direction, and a tiny flow model whose samples move towards what the reward prefers."""
import torch
import torch.nn as nn

from dew_b200.objectives.base import Step
from dew_b200.objectives.rl.nft import DiffusionNFT, optimality


class Velocity(nn.Module):
    def __init__(self, dim=2, hidden=64):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(dim + 1, hidden), nn.SiLU(), nn.Linear(hidden, hidden), nn.SiLU(), nn.Linear(hidden, dim))

    def forward(self, x, t):
        return self.net(torch.cat([x, t[:, None].expand(x.shape[0], 1)], -1))


def sample(model, n, steps=20, generator=None):
    x = torch.randn(n, 2, generator=generator)
    grid = torch.linspace(1.0, 0.0, steps + 1)
    with torch.no_grad():
        for i in range(steps):
            x = x - (grid[i] - grid[i + 1]) * model(x, grid[i].expand(n))
    return x


def test_optimality_and_the_sign_of_the_update():
    r = optimality(torch.tensor([1.0, 0.0, 3.0, 3.0]), group=2)
    assert r[0] > 0.5 > r[1] and r[2] == r[3] == 0.5 and float(r.min()) >= 0 and float(r.max()) <= 1
    torch.manual_seed(0)
    model = Velocity()
    obj = DiffusionNFT(model, group=2, beta=1.0)
    x0 = torch.randn(2, 2)
    step = Step(step=0, key=3)
    # with no old policy yet and beta 1, v+ = v_theta and v- = 2 v_old - v_theta: the rewarded image's regression error falls along the
    # negative gradient, the other's rises
    batch = {"x0": x0, "rewards": torch.tensor([1.0, -1.0])}
    stats, aux = obj.loss(None, batch, step)
    grads = torch.autograd.grad(stats.total, list(model.parameters()))
    t = step.sample("nft_t", (), 2, kind="uniform").float()
    eps = step.sample("nft_eps", (2,), 2).float()
    x_t, target = (1 - t[:, None]) * x0 + t[:, None] * eps, eps - x0

    def errors():
        with torch.no_grad():
            return (model(x_t, t) - target).pow(2).mean(1)
    before = errors()
    with torch.no_grad():
        for p, g in zip(model.parameters(), grads):
            p -= 1e-3 * g
    after = errors()
    assert after[0] < before[0] and after[1] > before[1]
    assert set(aux.metrics) == {"reward", "optimality", "policy_gap"}


def test_samples_move_towards_the_rewarded_side():
    torch.manual_seed(0)
    model = Velocity()
    opt = torch.optim.Adam(model.parameters(), lr=2e-3)
    g = torch.Generator().manual_seed(1)
    for i in range(300):                                         # pre-train on a unit Gaussian blob at the origin
        x0 = torch.randn(128, 2, generator=g) * 0.5
        t, eps = torch.rand(128, generator=g), torch.randn(128, 2, generator=g)
        loss = (model((1 - t[:, None]) * x0 + t[:, None] * eps, t) - (eps - x0)).pow(2).mean()
        opt.zero_grad(), loss.backward(), opt.step()
    start = float(sample(model, 512, generator=g)[:, 0].mean())
    obj = DiffusionNFT(model, group=8, beta=1.0, old_decay=0.9)
    opt = torch.optim.Adam(model.parameters(), lr=5e-4)
    for i in range(120):
        x0 = sample(model, 64, generator=g)
        batch = {"x0": x0, "rewards": x0[:, 0].clone()}              # reward: be to the right
        stats, _ = obj.loss(None, batch, Step(step=i, key=i))       # (no weight average here: the trained weights stand in for the old policy)
        opt.zero_grad()
        (stats.total / stats.mass).backward()
        opt.step()
    end = float(sample(model, 512, generator=g)[:, 0].mean())
    assert end > start + 0.3, (start, end)
