"""Reinforcement learning with a verifiable reward (GRPO): a small byte-level policy learns to answer single-digit sums.
Each round draws a group of completions per prompt from the rollout server, scores them with a checker, and takes policy
gradient steps on the group-normalised advantages.  Counterpart of the reference's examples/train_rlvr.py.

    python examples/train_rlvr.py [--rounds 30] [--device cuda]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.inference.rollouts import NativeRolloutServer, rescore
from dew_b200.inference.serving import Server
from dew_b200.models import CausalTransformer
from dew_b200.objectives.lm import LMObjective
from dew_b200.objectives.rl.policy import GRPO
from dew_b200.sampling.text import Sampling
from dew_b200.utils.trees import module_variables


def problems(g, n):
    a, b = torch.randint(0, 5, (n,), generator=g), torch.randint(0, 5, (n,), generator=g)
    return [(f"{int(x)}+{int(y)}=".encode(), str(int(x + y)).encode()) for x, y in zip(a, b)]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rounds", type=int, default=30)
    ap.add_argument("--pretrain", type=int, default=150)
    ap.add_argument("--group", type=int, default=4)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    model = CausalTransformer(vocab_size=256, emb_features=64, num_layers=2, num_heads=2, head_dim=32, mlp_features=128, max_seq_len=16,
                              qk_norm=False).to(dev)
    # a short supervised warm start so that some sampled answers are right (the reward needs a signal to amplify)
    sft = dew.Trainer(LMObjective(model, 5, ema_decay=None), dew.OptimConfig(learning_rate=3e-3), key=0)
    rows = [torch.tensor(list(q + a.ljust(2, b"\n")))[:6] for q, a in problems(g, 2048)]
    data = [{"tokens": torch.stack(rows[i:i + 64]).to(dev)} for i in range(0, 2048, 64)]
    sft.fit(data * (args.pretrain // len(data) + 1), steps=args.pretrain, log_every=10 ** 6)
    objective = GRPO(model, group=args.group, clip=0.2, kl=0.0)
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=3e-4), key=1)
    sampling = Sampling(temperature=1.0)
    history, state = [], None
    with NativeRolloutServer(Server(model, slots=32, capacity=16, sampling=sampling)) as server:
        for r in range(args.rounds):
            batch = problems(g, 8)
            futures = [server.submit(list(q), 2, key=r * 1000 + i * args.group + k, sampling=sampling)
                       for i, (q, _) in enumerate(batch) for k in range(args.group)]
            draws = [f.result(timeout=300) for f in futures]
            answers = [a for _, a in batch for _ in range(args.group)]
            rewards = torch.tensor([1.0 if bytes(d.tokens).rstrip(b"\n")[:len(a)] == a and len(bytes(d.tokens).rstrip(b"\n")) == len(a) else 0.0
                                    for d, a in zip(draws, answers)])
            old = rescore(model, None, draws)
            width = max(len(d.prompt) + len(d.tokens) for d in draws)
            tokens = torch.zeros(len(draws), width, dtype=torch.long)
            mask = torch.zeros(len(draws), width)
            old_lp = torch.zeros(len(draws), width - 1)
            for i, d in enumerate(draws):
                row = d.prompt + d.tokens
                tokens[i, :len(row)] = torch.tensor(row)
                mask[i, len(d.prompt):len(row)] = 1
                old_lp[i, len(d.prompt) - 1:len(row) - 1] = old[i].cpu()
            step_batch = {"tokens": tokens.to(dev), "mask": mask.to(dev), "rewards": rewards.to(dev), "old_logprobs": old_lp.to(dev)}
            state = trainer.fit([step_batch] * 2, state=state, steps=2 * (r + 1), log_every=10 ** 6)
            server.load(module_variables(model), r + 1)
            history.append(float(rewards.mean()))
    k = max(1, len(history) // 4)
    print(f"mean reward: first rounds {sum(history[:k]) / k:.2f} -> last rounds {sum(history[-k:]) / k:.2f}")
    return history


if __name__ == "__main__":
    main()
