"""Decisions as a model's output: a small decoder answers typed questions about a record (here: about an integer written in
digits), its answers are calibrated on held-out records (temperature, histogram binning), and low-confidence answers are routed
to a fallback (abstention) so that the answered ones meet an error target.  Counterpart of the reference's
examples/route_decisions.py.

    python examples/route_decisions.py [--steps 300] [--device cpu]
"""
import argparse
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.decision import (Budget, Choice, Decide, DecisionModel, DecisionObjective, Example, JointSchemaHead, Layout, LogLoss, Noul,
                               Score, measure)
from dew_b200.models import CausalTransformer

QUESTIONS = {"parity": Choice("is the number even or odd", ["even", "odd"]),
             "half": Noul("is the number at least 500"),
             "size": Score("how large is the number", ["below 334", "334 to 667", "668 and above"])}


def records(n, seed):
    g = np.random.default_rng(seed)
    return [Example(f"{int(v):03d}", QUESTIONS, {"parity": int(v % 2), "half": bool(v >= 500), "size": int(min(2, v // 334))})
            for v in g.integers(0, 1000, n)]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    layout = Layout(shape="joint", max_len=224, head_max_len=200)
    backbone = CausalTransformer(vocab_size=260, emb_features=64, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=32, mlp_features=128,
                                 max_seq_len=256)
    model = DecisionModel(backbone, JointSchemaHead(64, layers=1)).to(dev)
    objective = DecisionObjective(model, layout, rule=LogLoss(), length=224)
    train, held = records(512, 0), records(256, 1)
    batches = [{k: v.to(dev) for k, v in objective.batch(train[i:i + 32]).items()} for i in range(0, len(train), 32)]
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0), tracker=dew.MemoryTracker())
    trainer.fit(batches * (args.steps // len(batches) + 1), steps=args.steps, log_every=max(1, args.steps // 5))
    report = measure([objective.decisions({k: v.to(dev) for k, v in objective.batch(held[i:i + 32]).items()}) for i in range(0, len(held), 32)])
    print("held-out: " + "  ".join(f"{k} {v:.3f}" for k, v in report.items()))
    task = Decide(model, layout, budget=Budget(tokens=4096, lengths=(224, 448)), device=dev).calibrated(held, bins=10, target_error=0.05, least=20)
    answered = right = 0
    fresh = records(128, 2)
    for ex, ans in zip(fresh, task.decide([{"state": e.state, "questions": e.questions} for e in fresh])):
        for name, a in ans.items():
            if not a.abstained:
                answered += 1
                right += int(np.argmax(a.probabilities) == int(np.argmax(ex.distribution(name))))
    total = len(fresh) * len(QUESTIONS)
    report.update(answered=answered / total, answered_accuracy=right / max(answered, 1))
    print(f"answered {answered} of {total} questions at accuracy {report['answered_accuracy']:.3f}; the rest go to the fallback")
    print(task.systemone({"state": "642", "questions": {n: q.wire() for n, q in QUESTIONS.items()}}, details=True))
    return report


if __name__ == "__main__":
    main()
