"""A physics-informed network for the viscous Burgers equation ``u_t + u u_x = nu u_xx`` on ``x in [-1, 1], t in [0, 1]``
with ``u(x, 0) = -sin(pi x)`` and ``u(+-1, t) = 0``, trained by damped Gauss-Newton (Levenberg-Marquardt) steps: every step
solves the normal equations of all residuals (PDE, initial and boundary conditions) in the network's few hundred weights.
Counterpart of the reference's examples/pinn_burgers.py.

    python examples/pinn_burgers.py [--steps 40] [--device cpu]
"""
import argparse
import math
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dew_b200.optim.gauss_newton import LevenbergMarquardt


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--nu", type=float, default=0.05)
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    dt = torch.float64
    net = nn.Sequential(nn.Linear(2, 16), nn.Tanh(), nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 1)).to(dev, dt)
    g = torch.Generator().manual_seed(0)
    interior = torch.stack([torch.rand(400, generator=g, dtype=dt) * 2 - 1, torch.rand(400, generator=g, dtype=dt)], 1).to(dev)
    x0 = torch.linspace(-1, 1, 64, dtype=dt, device=dev)
    initial = torch.stack([x0, torch.zeros_like(x0)], 1)
    tb = torch.linspace(0, 1, 32, dtype=dt, device=dev)
    boundary = torch.cat([torch.stack([-torch.ones_like(tb), tb], 1), torch.stack([torch.ones_like(tb), tb], 1)])

    def residuals(params):
        u = lambda p: torch.func.functional_call(net, params, (p[None],))[0, 0]
        du = torch.func.grad(u)
        d2u_xx = lambda p: torch.func.grad(lambda q: du(q)[0])(p)[0]
        uv = torch.func.vmap(u)(interior)
        g1 = torch.func.vmap(du)(interior)
        uxx = torch.func.vmap(d2u_xx)(interior)
        pde = g1[:, 1] + uv * g1[:, 0] - args.nu * uxx
        ic = torch.func.vmap(u)(initial) + torch.sin(math.pi * x0)
        bc = torch.func.vmap(u)(boundary)
        return torch.cat([pde, 3.0 * ic, 3.0 * bc])

    lm = LevenbergMarquardt(damping=1e-2)
    history = []
    for step in range(args.steps):
        info = lm.step(net, residuals)
        history.append(info["loss"])
    print(f"sum of squared residuals: {history[0]:.4f} -> {history[-1]:.6f} after {args.steps} steps (damping {lm.damping:.2e})")
    return history


if __name__ == "__main__":
    main()
