"""Train a decoder-only language model (dense, mixture-of-experts or a recurrent hybrid) on byte tokens, evaluate its
perplexity and generate from it.  Counterpart of the reference's examples/train_lm.py.

    python examples/train_lm.py [--kind dense|moe|hybrid|mamba2] [--steps 200] [--device cuda]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.models import CausalTransformer
from dew_b200.models.causal_transformer import Mixture
from dew_b200.objectives.lm import LMObjective
from dew_b200.sampling.text import Sampling, generate

TEXT = ("it was the best of times, it was the worst of times, it was the age of wisdom, it was the age of foolishness, "
        "it was the epoch of belief, it was the epoch of incredulity. ")


def build(kind: str, dev, head_dim: int):
    common = dict(vocab_size=256, emb_features=128, num_layers=4, num_heads=2, head_dim=head_dim, mlp_features=256, max_seq_len=128,
                  qk_norm=False)
    if kind == "moe":
        return CausalTransformer(mixture=Mixture(experts=8, top_k=2, expert_features=128, shared_features=128), **common)
    if kind == "hybrid":
        return CausalTransformer(layer_types=("gdn", "gdn", "gdn", "attention"),
                                 mixer_options=dict(num_k_heads=1, num_v_heads=1, head_k_dim=128, head_v_dim=128), **common)
    if kind == "mamba2":
        return CausalTransformer(layer_types=("mamba2", "attention"), mixer_options=dict(state_dim=128, head_dim=64), **common)
    return CausalTransformer(**common)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="dense", choices=["dense", "moe", "hybrid", "mamba2"])
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    tokens = torch.tensor(list((TEXT * 300).encode()), dtype=torch.long)
    windows = tokens[: (len(tokens) // 129) * 129].view(-1, 129)
    train, held = windows[:-8], windows[-8:]
    model = build(args.kind, dev, 64).to(dev)
    objective = LMObjective(model, 128, balance=0.01 if args.kind == "moe" else None)
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=2e-3, clip_grads=1.0), tracker=dew.MemoryTracker(),
                          checkpoints=dew.Checkpoints(args.out, keep=dew.Keep(2)) if args.out else None,
                          param_dtype=torch.bfloat16 if dev.type == "cuda" else None)
    state = trainer.fit(dew.Memory({"tokens": train}).shuffle(0).repeat().batched(16), steps=args.steps, log_every=max(1, args.steps // 5))
    losses = [round(r["loss"], 3) for r in trainer.tracker.rows if "loss" in r]
    ev = trainer.evaluate(state, dew.Memory({"tokens": held}).batched(8))
    print(f"{args.kind}: loss {losses}, held-out perplexity {ev.get('perplexity', float('nan')):.2f}")
    prompt = list("it was the ".encode())
    out = generate(model, None, [prompt], 40, sampling=Sampling(temperature=0.0))
    print("greedy:", bytes(out.new_tokens(0).tolist()).decode(errors="replace"))
    return losses


if __name__ == "__main__":
    main()
