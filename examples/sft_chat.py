"""Supervised fine-tuning on conversations: messages are rendered with a chat template, every token carries its speaker's
role, and the objective scores the assistant's tokens only.  After training, the model answers a held-out prompt through
``render_prompt`` + ``generate``.  Counterpart of the reference's examples/sft_*.py (without a pretrained checkpoint: the
small decoder here starts from scratch on a toy task - answer with the colour word of the question upper-cased).

    python examples/sft_chat.py [--steps 300] [--device cuda]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.data import ByteTokenizer
from dew_b200.data.chat import Role, chat_batch, render_prompt
from dew_b200.models import CausalTransformer
from dew_b200.objectives.lm import LMObjective
from dew_b200.sampling.text import Sampling, generate

COLOURS = ["red", "green", "blue", "pink", "grey", "gold"]


def conversation(colour: str, answer: bool = True):
    msgs = [{"role": "system", "content": "shout the colour"}, {"role": "user", "content": f"colour: {colour}"}]
    return msgs + ([{"role": "assistant", "content": colour.upper()}] if answer else [])


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    tok = ByteTokenizer()
    model = CausalTransformer(vocab_size=tok.vocab_size, emb_features=96, num_layers=3, num_heads=4, num_kv_heads=2, head_dim=24, mlp_features=192,
                              max_seq_len=192, qk_norm=False).to(dev)
    train = COLOURS[:5]                                                       # "gold" is held out
    batch = chat_batch(tok, [conversation(c) for c in train] * 4, seq_len=160, pad_id=tok.pad_id)
    batch = {k: v.to(dev) for k, v in batch.items()}
    objective = LMObjective(model, 160, ema_decay=None, loss_role=int(Role.ASSISTANT), pad_id=tok.pad_id)
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=2e-3, clip_grads=1.0), key=0, tracker=dew.MemoryTracker())
    trainer.fit([batch] * args.steps, steps=args.steps, log_every=max(1, args.steps // 5))
    losses = [r["loss"] for r in trainer.tracker.rows if "loss" in r]
    answers = {}
    for c in COLOURS:
        prompt = render_prompt(tok, conversation(c, answer=False)).tolist()
        g = generate(model, None, [prompt], 18, sampling=Sampling(temperature=0.0))
        text = tok.decode([int(t) for t in g.new_tokens(0)])
        answers[c] = text.split("<|im_end|>")[0]
    right = sum(answers[c] == c.upper() for c in train)
    print(f"loss {losses[0]:.3f} -> {losses[-1]:.3f}; {right} of {len(train)} trained colours answered exactly; held-out 'gold' -> {answers['gold']!r}")
    return losses, right, answers


if __name__ == "__main__":
    main()
