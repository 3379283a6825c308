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


# ================================================================================================ a scoring server
# Requests that are answered by scoring rows (log-likelihoods of continuations, a decision model's option logits, a reward
# model's scores) rather than by generating: each request is admitted into rows, rows of many requests are scored together in
# passes, and a request is answered when all its rows are.  Reference: src/dew/inference/scoring.py (``Scoring``,
# ``ScoringRequest``, ``ScoringServer``: ``submit`` / ``run`` / ``reload``, per-request refusals, ``Metered``).
import threading
import time
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Generic, Optional, TypeVar


@dataclass
class ScoringRequest:
    rows: tuple                 # what the forward scores, one output each
    payload: Any = None         # what ``answer`` needs beside the outputs


class Scoring:
    """What a scoring server serves.  ``admit`` turns a request into rows (raising ``ValueError`` to refuse it: the refusal is
    that request's alone); ``forward`` scores a list of rows and returns one output per row, cutting them into passes as its
    budget demands; ``answer`` builds the request's result from its rows' outputs."""

    def admit(self, request: Any) -> ScoringRequest:
        raise NotImplementedError

    def forward(self, rows: list) -> list:
        raise NotImplementedError

    def answer(self, payload: Any, outputs: list) -> Any:
        raise NotImplementedError

    def metrics(self) -> Dict[str, float]:
        return {}


class ScoringServer:
    """``submit(request) -> Future``; ``run()`` scores everything pending; ``start()`` serves from a thread, scoring a batch when
    ``max_rows`` rows wait or the oldest has waited ``max_wait`` seconds.  ``reload(scoring)`` swaps the task (its weights and its
    calibration together) between passes, never inside one."""

    def __init__(self, scoring: Scoring, max_rows: int = 256, max_wait: float = 0.005):
        self.scoring, self.max_rows, self.max_wait = scoring, max_rows, max_wait
        self._pending: list = []                  # (ScoringRequest, Future, admitted-at)
        self._lock = threading.Lock()
        self._wake = threading.Condition(self._lock)
        self._thread: Optional[threading.Thread] = None
        self._stop = False
        self.requests = self.refused = self.rows_scored = self.passes = 0
        self.busy_s = 0.0

    def submit(self, request: Any) -> Future:
        """Admit ``request`` now (a refusal raises here, before anything is queued) and answer it in a later pass."""
        try:
            admitted = self.scoring.admit(request)
        except ValueError:
            with self._lock:
                self.refused += 1
            raise
        fut: Future = Future()
        with self._wake:
            self._pending.append((admitted, fut, time.perf_counter()))
            self.requests += 1
            self._wake.notify()
        return fut

    def _take(self) -> list:
        with self._lock:
            taken, rows = [], 0
            while self._pending and (not taken or rows + len(self._pending[0][0].rows) <= self.max_rows):
                item = self._pending.pop(0)
                taken.append(item)
                rows += len(item[0].rows)
            return taken

    def _score(self, taken: list) -> None:
        scoring = self.scoring                    # one task for the whole pass, whatever ``reload`` does meanwhile
        began = time.perf_counter()
        rows = [r for adm, _, _ in taken for r in adm.rows]
        try:
            outputs = scoring.forward(rows) if rows else []
        except Exception as e:                    # a failed pass fails its requests, not the server
            for _, fut, _ in taken:
                fut.set_exception(e)
            return
        at = 0
        for adm, fut, _ in taken:
            n = len(adm.rows)
            try:
                fut.set_result(scoring.answer(adm.payload, outputs[at:at + n]))
            except Exception as e:
                fut.set_exception(e)
            at += n
        self.rows_scored += len(rows)
        self.passes += 1
        self.busy_s += time.perf_counter() - began

    def run(self) -> None:
        while True:
            taken = self._take()
            if not taken:
                return
            self._score(taken)

    def reload(self, scoring: Scoring) -> None:
        with self._lock:
            self.scoring = scoring

    # -- serving from a thread
    def _loop(self) -> None:
        while True:
            with self._wake:
                while not self._stop and not self._pending:
                    self._wake.wait(0.1)
                if self._stop and not self._pending:
                    return
                oldest = self._pending[0][2]
                rows = sum(len(a.rows) for a, _, _ in self._pending)
                wait = self.max_wait - (time.perf_counter() - oldest)
                if rows < self.max_rows and wait > 0 and not self._stop:
                    self._wake.wait(wait)
            taken = self._take()
            if taken:
                self._score(taken)

    def start(self) -> "ScoringServer":
        if self._thread is None:
            self._stop = False
            self._thread = threading.Thread(target=self._loop, name="scoring-server", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def metrics(self) -> Dict[str, float]:
        return {"requests": float(self.requests), "refused": float(self.refused), "rows": float(self.rows_scored), "passes": float(self.passes),
                "rows_per_pass": self.rows_scored / max(1, self.passes), "busy_s": self.busy_s, **self.scoring.metrics()}


class LikelihoodScoring(Scoring):
    """``score`` as a served task: a request is ``(context ids, [continuation ids, ...])``, its answer the per-continuation
    ``(log-likelihood, tokens, greedy)`` triples."""

    def __init__(self, model, pad_id: int = 0, batch: int = 16):
        self.model, self.pad_id, self.batch = model, pad_id, batch

    def admit(self, request):
        context, continuations = request
        if not continuations or any(len(c) == 0 for c in continuations):
            raise ValueError("a likelihood request needs at least one non-empty continuation")
        return ScoringRequest(tuple((tuple(context), tuple(c)) for c in continuations))

    def forward(self, rows):
        return score(self.model, [c for c, _ in rows], [k for _, k in rows], self.pad_id, self.batch)

    def answer(self, payload, outputs):
        return list(outputs)
