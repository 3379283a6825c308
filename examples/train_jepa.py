"""Train an image JEPA: a context encoder and predictor regress the EMA target encoder's features of masked blocks, then
a linear probe reads the frozen encoder.  Counterpart of the reference's examples/train_jepa.py.

    python examples/train_jepa.py [--steps 200] [--device cuda]
"""
import argparse
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.objectives.jepa import JepaModel, JepaObjective, MultiBlockMask


class Encoder(nn.Module):
    """Patch tokens [B, T, p*p*3] -> [B, T, d] with learned positions and a small transformer."""

    def __init__(self, tokens: int, patch_dim: int, d: int = 64, layers: int = 2, heads: int = 4):
        super().__init__()
        self.proj = nn.Linear(patch_dim, d)
        self.pos = nn.Parameter(torch.zeros(tokens, d))
        self.blocks = nn.TransformerEncoder(nn.TransformerEncoderLayer(d, heads, 4 * d, dropout=0.0, batch_first=True, norm_first=True), layers)

    def forward(self, x):
        return self.blocks(self.proj(x) + self.pos[None])


def patches(images: torch.Tensor, p: int) -> torch.Tensor:
    B, H, W, C = images.shape
    return images.reshape(B, H // p, p, W // p, p, C).permute(0, 1, 3, 2, 4, 5).reshape(B, (H // p) * (W // p), p * p * C)


def synthetic(n: int, g: torch.Generator):
    """Two classes of 32 x 32 images: horizontal or vertical stripes with a random phase and noise."""
    labels = torch.randint(0, 2, (n,), generator=g)
    phase = torch.rand(n, generator=g) * 6.283
    axis = torch.arange(32).float()
    wave = torch.sin(axis[None] * 0.8 + phase[:, None])                        # [n, 32]
    img = torch.where(labels[:, None, None].bool(), wave[:, :, None].expand(n, 32, 32), wave[:, None, :].expand(n, 32, 32))
    img = img[..., None].expand(n, 32, 32, 3) + 0.1 * torch.randn(n, 32, 32, 3, generator=g)
    return img, labels


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    p, grid = 4, (8, 8)
    tokens, patch_dim, d = grid[0] * grid[1], p * p * 3, 64
    model = JepaModel(Encoder(tokens, patch_dim, d), Encoder(tokens, d, d, layers=1), d).to(dev)
    objective = JepaObjective(model, MultiBlockMask(grid=grid, targets=2), momentum=0.99)
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=1e-3), key=0, tracker=dew.MemoryTracker())
    images, labels = synthetic(512, g)
    data = [{"sample": patches(images[i:i + 32], p).to(dev)} for i in range(0, 512, 32)]
    state = trainer.fit(data * (args.steps // len(data) + 1), steps=args.steps, log_every=max(1, args.steps // 10))
    losses = [r["loss"] for r in trainer.tracker.rows if "loss" in r]
    # linear probe on the mean-pooled features of the frozen context encoder
    with torch.no_grad():
        feats = model(patches(images, p).to(dev)).mean(1).float().cpu()
    probe = torch.linalg.lstsq(torch.cat([feats, torch.ones(len(feats), 1)], 1)[:384], torch.nn.functional.one_hot(labels[:384], 2).float()).solution
    acc = float(((torch.cat([feats, torch.ones(len(feats), 1)], 1)[384:] @ probe).argmax(1) == labels[384:]).float().mean())
    print(f"step {state.step}: loss {losses[0]:.4f} -> {losses[-1]:.4f}; linear probe accuracy {acc:.2f}")
    return losses, acc


if __name__ == "__main__":
    main()
