"""Train a pixel-space diffusion transformer with the EDM objective (or flow matching) on synthetic images, keep EMA
weights, checkpoint, restore and sample a grid with a second-order solver.  Counterpart of the reference's
examples/train_diffusion.py and examples/train_flowers.py.

    python examples/train_diffusion.py [--process edm|flow] [--steps 100] [--device cuda]
"""
import argparse
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.models import SimpleDiT
from dew_b200.objectives.diffusion import DiffusionObjective


def blobs(n: int, size: int, seed: int) -> torch.Tensor:
    """Synthetic images: one soft coloured disc per image on a dark background, values in [-1, 1]."""
    g = torch.Generator().manual_seed(seed)
    yy, xx = torch.meshgrid(torch.linspace(-1, 1, size), torch.linspace(-1, 1, size), indexing="ij")
    cx, cy = torch.rand(n, generator=g) - 0.5, torch.rand(n, generator=g) - 0.5
    colour = torch.rand(n, 3, generator=g)
    disc = torch.exp(-((xx[None] - cx[:, None, None]) ** 2 + (yy[None] - cy[:, None, None]) ** 2) / 0.08)
    return (disc[..., None] * colour[:, None, None, :]) * 2 - 1


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--process", default="edm", choices=["edm", "flow"])
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    model = SimpleDiT(patch_size=4, emb_features=128, num_layers=4, num_heads=2).to(dev)
    process = dew.EDM(regime="pixel") if args.process == "edm" else dew.Flow()
    objective = DiffusionObjective(model, process, dew.InputSpec(dew.Field("sample", (32, 32, 3))), ema_decay=0.995)
    out = tempfile.mkdtemp(prefix="dewb_diffusion_")
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=2e-4), tracker=dew.MemoryTracker(), checkpoints=dew.Checkpoints(out, keep=dew.Keep(1)))
    data = dew.Memory({"sample": blobs(256, 32, 0)}).shuffle(0).repeat().batched(16)
    state = trainer.fit(data, steps=args.steps, log_every=max(1, args.steps // 4))
    losses = [round(r["loss"], 4) for r in trainer.tracker.rows if "loss" in r]
    restored = trainer.checkpoints.restore(state)
    solver = dew.Heun() if args.process == "edm" else dew.Euler()
    grid = objective.generate(restored.averaged, (8, 32, 32, 3), key=0, steps=12, solver=solver)
    print(f"{args.process}: loss {losses}; samples {tuple(grid.shape)} in [{float(grid.min()):.2f}, {float(grid.max()):.2f}] from EMA weights at step {restored.step}")
    return losses


if __name__ == "__main__":
    main()
