"""Adapter to the interface evaluation harnesses drive a language model through (EleutherAI's lm-evaluation-harness ``LM``):
``loglikelihood``, ``loglikelihood_rolling`` and ``generate_until`` over requests whose ``.args`` hold the strings.

The adapter does not import the harness: it is a plain object with the three methods, so ``lm_eval.simple_evaluate(model=
HarnessModel(...), tasks=[...])`` works where the harness is installed, and the methods can be called directly where it is
not.  Scoring is ``dew_b200.inference.scoring.score`` (one padded batch per group of requests); generation is the library's
``generate`` with the request's stop strings and token budget.

Reference: src/dew/eval (lm-eval harness adapter over the serving tasks).
"""
from __future__ import annotations

from typing import Any, List, Sequence, Tuple

import torch

from ..inference.scoring import score
from ..sampling.text import Sampling, generate


def _args(request: Any) -> tuple:
    return tuple(request.args) if hasattr(request, "args") else tuple(request)


class HarnessModel:
    def __init__(self, model: torch.nn.Module, tokenizer, *, max_length: int = 2048, batch_size: int = 16, bos_id: int = None,
                 max_gen_tokens: int = 256):
        self.model, self.tokenizer = model, tokenizer
        self.max_length, self.batch_size, self.max_gen_tokens = max_length, batch_size, max_gen_tokens
        self.bos_id = bos_id if bos_id is not None else getattr(tokenizer, "bos_id", None)

    # -- tokenisation -------------------------------------------------------------------------------------------
    def _encode(self, text: str) -> List[int]:
        return list(self.tokenizer.encode(text))

    def _pair(self, context: str, continuation: str) -> Tuple[List[int], List[int]]:
        """Tokenise context + continuation together and split at the context's length, so that a tokenizer that merges
        across the boundary scores the tokens the model would really see; trailing spaces of the context move to the
        continuation (the harness's convention)."""
        n_spaces = len(context) - len(context.rstrip())
        if n_spaces:
            continuation, context = context[-n_spaces:] + continuation, context[:-n_spaces]
        whole, ctx = self._encode(context + continuation), self._encode(context)
        ctx_ids, con_ids = whole[:len(ctx)], whole[len(ctx):]
        if not ctx_ids:
            ctx_ids = [self.bos_id if self.bos_id is not None else 0]
        over = len(ctx_ids) + len(con_ids) - self.max_length          # keep the continuation, drop the oldest context
        if over > 0:
            ctx_ids = ctx_ids[over:] or ctx_ids[-1:]
        return ctx_ids, con_ids

    # -- the three calls ----------------------------------------------------------------------------------------
    def loglikelihood(self, requests: Sequence[Any]) -> List[Tuple[float, bool]]:
        pairs = [self._pair(*_args(r)[:2]) for r in requests]
        res = score(self.model, [p[0] for p in pairs], [p[1] for p in pairs], batch=self.batch_size)
        return [(lp, greedy) for lp, _, greedy in res]

    def loglikelihood_rolling(self, requests: Sequence[Any]) -> List[float]:
        """Whole-document log-likelihood: windows of ``max_length`` tokens, each scored given one token of context."""
        out = []
        for r in requests:
            ids = self._encode(_args(r)[0])
            first = self.bos_id if self.bos_id is not None else (ids[0] if ids else 0)
            if self.bos_id is None:
                ids = ids[1:]
            total, prev = 0.0, first
            for lo in range(0, len(ids), self.max_length - 1):
                win = ids[lo:lo + self.max_length - 1]
                total += score(self.model, [[prev]], [win], batch=1)[0][0]
                prev = win[-1]
            out.append(total)
        return out

    def generate_until(self, requests: Sequence[Any]) -> List[str]:
        outs = []
        for r in requests:
            context, kwargs = _args(r)[0], (_args(r)[1] if len(_args(r)) > 1 else {})
            until = kwargs.get("until", [])
            until = [until] if isinstance(until, str) else list(until)
            budget = int(kwargs.get("max_gen_toks", self.max_gen_tokens))
            temp = float(kwargs.get("temperature", 0.0)) if kwargs.get("do_sample", False) else 0.0
            ids = self._encode(context)[-(self.max_length - budget):]
            g = generate(self.model, None, [ids], budget, sampling=Sampling(temperature=temp))
            text = self.tokenizer.decode([int(t) for t in g.new_tokens(0)])
            for stop in until:
                if stop and stop in text:
                    text = text[: text.index(stop)]
            outs.append(text)
        return outs
