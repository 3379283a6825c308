"""Train a small language model without backpropagation: node perturbation estimates every layer's gradient from pairs of
jittered forward passes (no gradient crosses a layer boundary), and the same model trained by backpropagation is the yardstick.
Counterpart of the reference's examples/forward_only_lm.py.

    python examples/forward_only_lm.py [--steps 300] [--draws 8] [--device cpu]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.models import CausalTransformer
from dew_b200.objectives.lm import LMObjective
from dew_b200.objectives.perturbation import NodePerturbation


def corpus(n: int, seq: int, g: torch.Generator) -> torch.Tensor:
    """Sequences from a fixed first-order Markov chain over 16 symbols: learnable structure with a known entropy floor."""
    table = torch.softmax(torch.randn(16, 16, generator=torch.Generator().manual_seed(7)) * 2.0, -1)
    rows = torch.zeros(n, seq + 1, dtype=torch.long)
    rows[:, 0] = torch.randint(0, 16, (n,), generator=g)
    for t in range(seq):
        rows[:, t + 1] = torch.multinomial(table[rows[:, t]], 1, generator=g).squeeze(1)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--draws", type=int, default=8)
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    g = torch.Generator().manual_seed(0)
    data = corpus(1024, 16, g)
    batches = [{"tokens": data[i:i + 64].to(dev)} for i in range(0, 1024, 64)]

    def model():
        torch.manual_seed(0)
        return CausalTransformer(vocab_size=16, emb_features=32, num_layers=1, num_heads=2, head_dim=16, mlp_features=64, max_seq_len=16, qk_norm=False).to(dev)

    results = {}
    for name, objective, lr in (("forward_only", lambda m: NodePerturbation(m, 16, sigma=1e-2, draws=args.draws), 1e-2),
                                ("backprop", lambda m: LMObjective(m, 16, ema_decay=None), 3e-3)):
        tracker = dew.MemoryTracker()
        trainer = dew.Trainer(objective(model()), dew.OptimConfig(learning_rate=lr, weight_decay=0.0), tracker=tracker)
        trainer.fit(batches * (args.steps // len(batches) + 1), steps=args.steps, log_every=max(1, args.steps // 6))
        results[name] = [r["loss"] for r in tracker.rows]
        print(f"{name:13s} loss " + " -> ".join(f"{l:.3f}" for l in results[name]))
    return results


if __name__ == "__main__":
    main()
