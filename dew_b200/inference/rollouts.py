"""Rollout servers for on-policy RL: one submission interface over the continuous-batching ``Server``.

``submit(prompt ids, ...)`` returns a future ``Draw`` with the sampled ids, whether the policy ended the draw itself and
the policy version it was submitted under.  ``load(variables, version)`` pushes new weights while generation keeps
running: the swap happens between two server steps, in-flight requests finish on whichever weights are resident when each
token is drawn, and a draw's ``version`` is the oldest weights that may have produced any of its tokens (the version
resident when it was submitted).  ``rescore`` gives the trainer's own per-token log-likelihoods of finished draws.

``NativeRolloutServer`` drives a ``Server`` on a background thread.  Remote engines (OpenAI-compatible completions
endpoints) implement the same three calls in ``dew_b200.inference.clients``.

Reference: src/dew/inference/rollouts.py (``Draw``, ``RolloutServer``, ``NativeRolloutServer``, ``check_ending``).
"""
from __future__ import annotations

import threading
from concurrent.futures import Future
from dataclasses import dataclass
from typing import Any, List, Optional, Sequence, Tuple

import torch

from ..sampling.text import Sampling
from .serving import Server, Ticket


@dataclass
class Draw:
    prompt: List[int]
    tokens: List[int]
    terminated: bool            # the policy ended the draw (EOS / stop) rather than the budget
    version: int                # oldest policy version that may have produced a token of this draw
    newest_version: int         # version resident when the draw finished (== version when no load happened meanwhile)

    @property
    def stale(self) -> bool:
        return self.newest_version != self.version


class RolloutServer:
    """The interface: ``submit`` -> Future[Draw], ``load`` new weights under a version, ``close``."""

    def submit(self, prompt: Sequence[int], max_new_tokens: int, *, key: int = 0, sampling: Optional[Sampling] = None) -> "Future[Draw]":
        raise NotImplementedError

    def load(self, variables: Any, version: int) -> None:
        raise NotImplementedError

    def close(self) -> None:
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class NativeRolloutServer(RolloutServer):
    def __init__(self, server: Server, version: int = 0):
        self.server, self.version = server, int(version)
        self._lock = threading.Condition()
        self._incoming: List[Tuple[Ticket, Future, int]] = []      # submitted, not yet handed to the server loop
        self._live: List[Tuple[Ticket, Future, int]] = []
        self._pending_load: Optional[Tuple[Any, int]] = None
        self._closing = False
        self._error: Optional[BaseException] = None
        self._thread = threading.Thread(target=self._loop, name="rollout-server", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ the interface
    def submit(self, prompt, max_new_tokens, *, key=0, sampling=None):
        fut: Future = Future()
        with self._lock:
            if self._closing:
                raise RuntimeError("the rollout server is closed")
            if self._error is not None:
                raise self._error
            prompt = [int(t) for t in prompt]
            if len(prompt) + max_new_tokens > self.server.capacity:
                raise ValueError(f"prompt of {len(prompt)} tokens + {max_new_tokens} new exceeds the row capacity {self.server.capacity}")
            self._incoming.append((Ticket(prompt, max_new_tokens, key, sampling), fut, self.version))
            self._lock.notify_all()
        return fut

    def load(self, variables, version: int) -> None:
        """Queue a weight swap; it is applied between two server steps.  Versions must not go backwards."""
        with self._lock:
            if version < self.version:
                raise ValueError(f"policy versions only grow: {version} after {self.version}")
            self._pending_load = (variables, int(version))
            self.version = int(version)
            self._lock.notify_all()

    def close(self) -> None:
        with self._lock:
            self._closing = True
            self._lock.notify_all()
        self._thread.join(timeout=60)

    # ------------------------------------------------------------------ the loop
    def _loop(self) -> None:
        resident = self.version
        try:
            while True:
                with self._lock:
                    while not (self._incoming or self._live or self._pending_load or self._closing):
                        self._lock.wait()
                    if self._closing and not self._live and not self._incoming:
                        return
                    incoming, self._incoming = self._incoming, []
                    load, self._pending_load = self._pending_load, None
                if load is not None:
                    self.server.reload(load[0])
                    resident = load[1]
                for ticket, fut, version in incoming:
                    ticket.submitted = self.server.clock()
                    self.server.queue.append(ticket)
                    self._live.append((ticket, fut, version))
                if self.server.busy:
                    self.server.step()
                still = []
                for ticket, fut, version in self._live:
                    if ticket.done:
                        if ticket.error is not None:
                            fut.set_exception(ticket.error)
                        else:
                            fut.set_result(Draw(ticket.prompt, list(ticket.tokens), bool(ticket.terminated), version, resident))
                    else:
                        still.append((ticket, fut, version))
                self._live = still
        except BaseException as exc:                      # fail every waiter rather than leave futures hanging
            with self._lock:
                self._error = exc
                waiting = self._live + self._incoming
                self._live, self._incoming = [], []
            for _, fut, _ in waiting:
                if not fut.done():
                    fut.set_exception(exc)


@torch.no_grad()
def rescore(model, variables, draws: Sequence[Draw], pad_id: int = 0) -> List[torch.Tensor]:
    """The trainer's own log-likelihood of every drawn token, one tensor per draw (``[len(tokens)]``), by one padded forward."""
    if not draws:
        return []
    rows = [d.prompt + d.tokens for d in draws]
    width = max(len(r) for r in rows)
    dev = next(model.parameters()).device
    tok = torch.full((len(rows), width), pad_id, dtype=torch.long, device=dev)
    for i, r in enumerate(rows):
        tok[i, :len(r)] = torch.tensor(r, device=dev)
    if variables is None:
        logits = model(tok[:, :-1])
    else:
        from ..utils.trees import variables_for_call
        logits = torch.func.functional_call(model, variables_for_call(model, variables), (tok[:, :-1],))
    logp = torch.log_softmax(logits.float(), -1).gather(-1, tok[:, 1:, None]).squeeze(-1)
    return [logp[i, len(d.prompt) - 1:len(d.prompt) - 1 + len(d.tokens)].clone() for i, d in enumerate(draws)]
