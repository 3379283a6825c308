"""Train a masked (discrete) diffusion language model - bidirectional transformer, MDLM objective - and sample text by
ancestral unmasking.  Counterpart of the reference's examples/train_masked_lm.py.

    python examples/train_masked_lm.py [--steps 200]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.objectives.discrete import MaskedDiffusionLM

MASK = 256


class BidirectionalLM(torch.nn.Module):
    def __init__(self, vocab: int = 257, d: int = 128, layers: int = 3, heads: int = 4, length: int = 64):
        super().__init__()
        self.embed = torch.nn.Embedding(vocab, d)
        self.pos = torch.nn.Parameter(torch.zeros(length, d))
        layer = torch.nn.TransformerEncoderLayer(d, heads, 4 * d, dropout=0.0, batch_first=True, norm_first=True)
        self.body = torch.nn.TransformerEncoder(layer, layers)
        self.head = torch.nn.Linear(d, vocab)

    def forward(self, tokens, **kw):
        return self.head(self.body(self.embed(tokens) + self.pos[: tokens.shape[1]]))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    text = ("all work and no play makes jack a dull boy. " * 400).encode()
    tokens = torch.tensor(list(text), dtype=torch.long)
    windows = tokens[: (len(tokens) // 64) * 64].view(-1, 64)
    model = BidirectionalLM().to(dev)
    objective = MaskedDiffusionLM(model, mask_id=MASK)
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=2e-3), tracker=dew.MemoryTracker())
    state = trainer.fit(dew.Memory({"tokens": windows}).shuffle(0).repeat().batched(32), steps=args.steps, log_every=max(1, args.steps // 4))
    rows = [r for r in trainer.tracker.rows if "loss" in r]
    print("loss:", [round(r["loss"], 3) for r in rows], "masked accuracy:", [round(r.get("masked_accuracy", float("nan")), 3) for r in rows])
    sample = objective.sample(state.variables, 2, 64, steps=16, generator=torch.Generator().manual_seed(0), device=dev)
    for row in sample.tolist():
        print("sample:", bytes(t for t in row if t < 256).decode(errors="replace"))
    return [r["loss"] for r in rows]


if __name__ == "__main__":
    main()
