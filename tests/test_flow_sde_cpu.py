"""Flow SDE transitions: closed forms, densities, trajectories and rescoring."""
import math

import pytest
import torch

from dew_b200.diffusion import presets
from dew_b200.sampling.flow import FlowSDE, GaussianTransition, flow_transition


def test_transition_closed_forms_and_limits():
    x, v = torch.randn(3, 4, 2), torch.randn(3, 4, 2)
    a, s, sn = 0.7, 0.6, 0.45
    tr = flow_transition(x, v, s, sn, noise_level=a)
    c, dt = a * a / (2 * (1 - s)), sn - s
    assert torch.allclose(tr.mean, x * (1 + c * dt) + v * (1 + c * (1 - s)) * dt, atol=1e-6)
    assert torch.allclose(tr.variance, torch.full((3,), a * a * s / (1 - s) * -dt), atol=1e-7)
    det = flow_transition(x, v, s, sn, noise_level=0.0)                # no noise: the Euler step of the ODE
    assert torch.allclose(det.mean, x + v * dt, atol=1e-6) and not bool(det.stochastic.any())
    assert torch.isnan(det.log_prob(det.mean)).all() and torch.equal(det.sample(0), det.mean)
    first = flow_transition(x, v, 1.0, 0.9, noise_level=a)             # at pure noise the denominator uses the next rate
    assert torch.isfinite(first.mean).all() and torch.allclose(first.variance, torch.full((3,), a * a * 1.0 / (1 - 0.9) * 0.1))
    assert torch.isnan(flow_transition(x, v, 0.3, 0.5).variance).all()  # rates must descend
    with pytest.raises(ValueError):
        flow_transition(x, v[:, :2], s, sn)


def test_density_matches_torch_normal_and_kl():
    mean, var = torch.randn(2, 5), torch.tensor([0.3, 1.7])
    tr = GaussianTransition(mean, var)
    value = tr.sample(3)
    ref = torch.distributions.Normal(mean, var.sqrt()[:, None]).log_prob(value).sum(1)
    assert torch.allclose(tr.log_prob(value), ref, atol=1e-5)
    other = mean + 0.5
    assert torch.allclose(tr.kl(other), torch.tensor([5 * 0.25 / (2 * 0.3), 5 * 0.25 / (2 * 1.7)]), atol=1e-6)


class _Velocity(torch.nn.Module):
    """A linear velocity field, so the marginals stay Gaussian and the test is exact enough."""

    def __init__(self):
        super().__init__()
        self.w = torch.nn.Parameter(torch.tensor(0.3))

    def forward(self, x, t, conditions=None):
        return self.w * x


def test_trajectory_records_and_rescores():
    process = presets.Flow()()
    model = _Velocity()
    den = process.denoiser(model, None, {})
    solver = FlowSDE(noise_level=0.7)
    x_T = torch.randn(4, 3, 2)
    traj = solver.trajectory(den, x_T, 6, key=11)
    assert traj.states.shape == (4, 6, 3, 2) and traj.log_probs.shape == (4, 5) and traj.times.shape == (6,)
    assert torch.equal(traj.states[:, 0], x_T) and traj.samples.shape == (4, 3, 2)
    assert bool(traj.stochastic[:, :-1].all())
    # rescoring a recorded transition under the same weights reproduces its density; under other weights it differs and
    # carries a gradient
    tr = solver.rescore(den, traj, 2)
    assert torch.allclose(tr.log_prob(traj.states[:, 3]), traj.log_probs[:, 2], atol=1e-4)
    with torch.no_grad():
        model.w.add_(0.2)
    lp = solver.rescore(den, traj, 2).log_prob(traj.states[:, 3])
    assert not torch.allclose(lp, traj.log_probs[:, 2], atol=1e-3)
    lp.sum().backward()
    assert model.w.grad is not None and float(model.w.grad.abs()) > 0
    # the same key draws the same trajectory
    again = solver.trajectory(den, x_T, 6, key=11)
    assert not torch.equal(again.states, traj.states)       # weights moved
    with pytest.raises(ValueError):
        solver.trajectory(den, x_T, 1)
    with pytest.raises(ValueError):
        FlowSDE().validate(presets.EDM(regime="pixel")())
