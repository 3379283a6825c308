"""Serve a decision model over HTTP: train a small model on typed questions about numbers (or load a saved task with ``--run``),
calibrate it, start the service, and answer a few requests through it the way a client would.  Counterpart of the reference's
examples/serve_decisions.py.

    python examples/serve_decisions.py [--steps 200] [--port 0] [--forever]
    curl -s localhost:PORT/v1/decide?details=1 -d '{"state": "642", "questions": {"even": {"type": "noul", "instructions": "is it even"}}}'
"""
import argparse
import json
import os
import sys
import urllib.request

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.decision import Budget, Decide, DecisionModel, DecisionObjective, JointSchemaHead, Layout, LogLoss
from dew_b200.decision.http import DecisionService
from dew_b200.models import CausalTransformer
from examples.route_decisions import QUESTIONS, records


def build(steps: int, device) -> Decide:
    torch.manual_seed(0)
    layout = Layout(shape="joint", max_len=224, head_max_len=200)
    backbone = CausalTransformer(vocab_size=260, emb_features=64, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=32, mlp_features=128, max_seq_len=256)
    model = DecisionModel(backbone, JointSchemaHead(64, layers=1)).to(device)
    objective = DecisionObjective(model, layout, rule=LogLoss(), length=224)
    train = records(512, 0)
    batches = [{k: v.to(device) for k, v in objective.batch(train[i:i + 32]).items()} for i in range(0, len(train), 32)]
    dew.Trainer(objective, dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0), tracker=dew.MemoryTracker()).fit(
        batches * (steps // len(batches) + 1), steps=steps, log_every=10 ** 9)
    return Decide(model, layout, budget=Budget(tokens=8192, lengths=(224, 448)), device=device).calibrated(records(256, 1), target_error=0.05)


def post(address, body, query=""):
    req = urllib.request.Request(f"http://{address[0]}:{address[1]}/v1/decide{query}", data=json.dumps(body).encode(), method="POST")
    with urllib.request.urlopen(req, timeout=60) as r:
        return json.loads(r.read())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--forever", action="store_true")
    args = ap.parse_args(argv)
    task = build(args.steps, torch.device(args.device))
    wire = {n: q.wire() for n, q in QUESTIONS.items()}
    with DecisionService(task, port=args.port) as service:
        print(f"serving on http://{service.address[0]}:{service.address[1]}")
        one = post(service.address, {"state": "642", "questions": wire}, "?details=1")
        many = post(service.address, [{"state": f"{v:03d}", "questions": wire} for v in (7, 250, 999)] + [{"state": "1", "questions": {}}])
        print(json.dumps(one["answers"]["parity"]), json.dumps(many[-1]))
        with urllib.request.urlopen(f"http://{service.address[0]}:{service.address[1]}/metrics", timeout=10) as r:
            metrics = r.read().decode()
        if args.forever:
            import time
            while True:
                time.sleep(3600)
    return one, many, metrics


if __name__ == "__main__":
    main()
