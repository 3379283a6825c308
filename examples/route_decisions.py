"""Decisions as a model's output: a small decoder answers typed questions about a record (here: about an integer written in
digits), the answers are calibrated by temperature on held-out records, and low-confidence records are routed to a fallback
(abstention) so that the answered ones meet an accuracy target.  Counterpart of the reference's examples/route_decisions.py.

    python examples/route_decisions.py [--steps 300] [--device cpu]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.decision.calibration import Abstention, Temperatures, binning
from dew_b200.decision.model import Decide
from dew_b200.decision.objective import DecisionObjective
from dew_b200.decision.questions import Choice
from dew_b200.models import CausalTransformer


def records(n, g):
    values = torch.randint(0, 1000, (n,), generator=g)
    states = [[1 + int(d) for d in f"{int(v):03d}"] for v in values]            # digit tokens 1..10
    answers = torch.stack([values % 2, (values >= 500).long(), (values % 5 == 0).long()], 1)
    return states, answers


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    questions = [Choice("parity", ("even", "odd")), Choice("half", ("low", "high")), Choice("multiple_of_five", ("no", "yes"))]
    backbone = CausalTransformer(vocab_size=16, emb_features=48, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=24, mlp_features=96, max_seq_len=16)
    task = Decide(backbone, questions, marker_id=15, max_len=8, width=32).to(dev)
    train_states, train_answers = records(1024, g)
    held_states, held_answers = records(256, g)
    tokens, pos = task.encode(train_states)
    batches = [{"tokens": tokens[i:i + 128].to(dev), "positions": pos[i:i + 128].to(dev), "answers": train_answers[i:i + 128].to(dev)}
               for i in range(0, 1024, 128)]
    trainer = dew.Trainer(DecisionObjective(task, rule="log"), dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0), tracker=dew.MemoryTracker())
    trainer.fit(batches * (args.steps // len(batches) + 1), steps=args.steps, log_every=max(1, args.steps // 5))
    ht, hp = task.encode(held_states)
    with torch.no_grad():
        logits = [l.cpu() for l in task.logits(ht.to(dev), hp.to(dev))]
    temps = Temperatures.fit(logits, held_answers)
    report = {}
    for qi, q in enumerate(questions):
        probs = torch.softmax(logits[qi] / temps.value[qi], -1)
        correct = probs.argmax(-1) == held_answers[:, qi]
        _, ece = binning(probs.max(-1).values, correct)
        coverage, accuracy = Abstention(0.9).coverage_accuracy(probs, held_answers[:, qi])
        report[q.name] = {"accuracy": float(correct.float().mean()), "ece": float(ece), "answered": float(coverage), "answered_accuracy": float(accuracy)}
        print(f"{q.name:18s} accuracy {report[q.name]['accuracy']:.2f}  ece {ece:.3f}  answered {coverage:.2f} of records at accuracy {accuracy:.2f}")
    return report


if __name__ == "__main__":
    main()
