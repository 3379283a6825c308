"""Score continuations by log-likelihood and serve a model with continuous batching: requests of different lengths arrive
over time, share a paged KV cache and a prefix cache, and stream their tokens.  Counterpart of the reference's
examples/evaluate_and_serve.py.

    python examples/evaluate_and_serve.py [--device cuda]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dew_b200.inference.scoring import score
from dew_b200.inference.serving import Server
from dew_b200.models import CausalTransformer
from dew_b200.nn.kv_cache import KVCache
from dew_b200.sampling.text import Sampling, generate


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=256, emb_features=128, num_layers=2, num_heads=2, head_dim=64, mlp_features=256, max_seq_len=256,
                              qk_norm=False).to(dev).eval()
    if dev.type == "cuda":
        model = model.to(torch.bfloat16)
    # 1. multiple-choice scoring: which continuation does the model find most likely?
    context = list(b"the capital of france is")
    choices = [list(b" paris"), list(b" london"), list(b" a fish")]
    scores = score(model, [context] * 3, choices)
    print("log-likelihoods:", [round(s, 2) for s, _, _ in scores])
    # 2. continuous batching: eight requests, a shared system prompt (prefix cache hits), paged KV
    server = Server(model, slots=4, capacity=128, kv_cache=KVCache(page_size=16, pages=64), sampling=Sampling(temperature=0.0))
    system = list(b"you are a helpful assistant. ")
    tickets = [server.submit(system + list(f"question {i}: ".encode()), max_new_tokens=8 + 2 * i, key=i) for i in range(8)]
    server.run()
    for i, t in enumerate(tickets):
        print(f"request {i}: {len(t.tokens)} tokens, first token after {1000 * (t.first_token_time or 0):.1f} ms")
    # the server's greedy tokens equal plain generation's
    ref = generate(model, None, [tickets[0].prompt], len(tickets[0].tokens), sampling=Sampling(temperature=0.0))
    same = ref.new_tokens(0).tolist() == list(tickets[0].tokens)
    print("server == generate:", same, "| prefix cache hits:", getattr(server.ledger, "hits", "n/a"))
    return same


if __name__ == "__main__":
    main()
