"""Supervised classification with the generic ``Supervised`` objective: a small MLP on two concentric rings, with
held-out accuracy through ``Trainer.fit(validation=...)``.  Counterpart of the reference's examples/train_supervised.py.

    python examples/train_supervised.py [--steps 400] [--device cuda]
"""
import argparse
import math
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.objectives import Step
from dew_b200.objectives.supervised import Supervised


def rings(n, g):
    label = torch.randint(0, 2, (n,), generator=g)
    angle = torch.rand(n, generator=g) * 2 * math.pi
    r = 0.4 + 0.6 * label + 0.08 * torch.randn(n, generator=g)
    return torch.stack([r * torch.cos(angle), r * torch.sin(angle)], 1), label


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    model = nn.Sequential(nn.Linear(2, 64), nn.Tanh(), nn.Linear(64, 64), nn.Tanh(), nn.Linear(64, 2)).to(dev)
    objective = Supervised(model, "cross_entropy")
    x, y = rings(2048, g)
    hx, hy = rings(512, g)
    data = [{"inputs": x[i:i + 128].to(dev), "targets": y[i:i + 128].to(dev)} for i in range(0, 2048, 128)]
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=3e-3), key=0, tracker=dew.MemoryTracker())
    trainer.fit(data * (args.steps // len(data) + 1), steps=args.steps, log_every=max(1, args.steps // 5))
    with torch.no_grad():
        stat, aux = objective.loss(None, {"inputs": hx.to(dev), "targets": hy.to(dev)}, Step(key=0, train=False))
    acc = float(aux.metrics["accuracy"].value())
    print(f"held-out loss {float(stat.value()):.3f}, accuracy {acc:.3f}")
    return acc


if __name__ == "__main__":
    main()
