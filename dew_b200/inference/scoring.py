"""Log-likelihood scoring of continuations (the primitive behind multiple-choice evaluation harnesses).

``score(model, contexts, continuations)`` returns, per pair, the summed log-probability of the continuation given the
context, its token count and whether the continuation is the greedy decode.  Pairs are right-padded into one batch;
on a GPU the forward takes this library's kernels like any other call of the model.
Reference: src/dew/inference/scoring.py (344 lines), src/dew/eval (lm-eval harness adapter).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


@torch.no_grad()
def score(model, contexts: Sequence[Sequence[int]], continuations: Sequence[Sequence[int]], pad_id: int = 0,
          batch: int = 16) -> List[Tuple[float, int, bool]]:
    dev = next(model.parameters()).device
    out: List[Tuple[float, int, bool]] = []
    for lo in range(0, len(contexts), batch):
        ctx, con = contexts[lo:lo + batch], continuations[lo:lo + batch]
        seqs = [list(c) + list(k) for c, k in zip(ctx, con)]
        T = max(len(s) for s in seqs)
        toks = torch.full((len(seqs), T), pad_id, dtype=torch.long)
        for i, s in enumerate(seqs):
            toks[i, :len(s)] = torch.tensor(s)
        logp = torch.log_softmax(model(toks.to(dev)).float(), -1).cpu()
        for i, (c, k) in enumerate(zip(ctx, con)):
            pos = torch.arange(len(c) - 1, len(c) + len(k) - 1)             # logits at t predict token t + 1
            tgt = torch.tensor(list(k))
            rows = logp[i, pos]
            out.append((float(rows.gather(-1, tgt[:, None]).sum()), len(k), bool((rows.argmax(-1) == tgt).all())))
    return out


def multiple_choice_accuracy(model, items: Sequence[Tuple[Sequence[int], Sequence[Sequence[int]], int]], normalize: bool = True) -> float:
    """``items``: (context, choices, answer index).  ``normalize`` divides by the choice length (acc_norm)."""
    right = 0
    for ctx, choices, answer in items:
        scores = score(model, [ctx] * len(choices), choices)
        vals = [s / max(n, 1) if normalize else s for s, n, _ in scores]
        right += int(max(range(len(vals)), key=vals.__getitem__) == answer)
    return right / max(len(items), 1)
