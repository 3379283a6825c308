"""One engine that serves kinds together.  A text server (continuous batching) and scoring servers (forward passes over batched rows)
would each run their own loop and meet on the device by chance; ``Engine`` owns the one loop that drives them, so their passes
alternate on one stream: a decode step of the text server, then one scoring pass per kind that has rows waiting, and so on while anything
is busy.  A long scoring queue therefore costs a generation one pass per step rather than its whole length, and neither kind starves.
``submit(kind, ...)`` forwards to the kind's own ``submit`` (a ``Ticket`` for text, a ``Future`` for scoring); ``reload`` swaps a kind's
task between passes; ``metrics`` merges the kinds' own under their names.

Reference: src/dew/inference/engine.py.
"""
from __future__ import annotations

import threading
import time
from typing import Any, Dict, Mapping, Optional


class Engine:
    def __init__(self, text=None, scoring: Optional[Mapping[str, Any]] = None, idle_wait: float = 0.002):
        self.text, self.scoring = text, dict(scoring or {})
        if text is None and not self.scoring:
            raise ValueError("an engine serves at least one kind")
        if "text" in self.scoring:
            raise ValueError("'text' names the generation server; call a scoring kind something else")
        self.idle_wait = idle_wait
        self._thread: Optional[threading.Thread] = None
        self._stop = False
        self.steps = {"text": 0, **{k: 0 for k in self.scoring}}

    @property
    def kinds(self):
        return (["text"] if self.text is not None else []) + list(self.scoring)

    def submit(self, kind: str, *args, **kwargs):
        if kind == "text":
            if self.text is None:
                raise KeyError(f"this engine serves no text; it serves {self.kinds}")
            return self.text.submit(*args, **kwargs)
        if kind not in self.scoring:
            raise KeyError(f"this engine serves no {kind!r}; it serves {self.kinds}")
        return self.scoring[kind].submit(*args, **kwargs)

    def busy(self) -> bool:
        return (self.text is not None and bool(self.text.busy)) or any(s._pending for s in self.scoring.values())

    def step(self) -> bool:
        """One round: a text step if generation is busy, then one pass of every scoring kind with rows waiting.  True if anything ran."""
        ran = False
        if self.text is not None and self.text.busy:
            self.text.step()
            self.steps["text"] += 1
            ran = True
        for name, server in self.scoring.items():
            taken = server._take()
            if taken:
                server._score(taken)
                self.steps[name] += 1
                ran = True
        return ran

    def run(self, max_rounds: Optional[int] = None) -> None:
        """Serve until nothing is busy (or ``max_rounds`` rounds)."""
        n = 0
        while self.busy() and (max_rounds is None or n < max_rounds):
            self.step()
            n += 1

    def reload(self, kind: str, task) -> None:
        (self.text if kind == "text" else self.scoring[kind]).reload(task)

    # -- serving from a thread
    def _loop(self) -> None:
        while not self._stop:
            if not self.step():
                time.sleep(self.idle_wait)

    def start(self) -> "Engine":
        if self._thread is None:
            self._stop = False
            self._thread = threading.Thread(target=self._loop, name="engine", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop = True
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def metrics(self) -> Dict[str, float]:
        out: Dict[str, float] = {f"rounds/{k}": float(v) for k, v in self.steps.items()}
        for name, server in self.scoring.items():
            out.update({f"{name}/{k}": v for k, v in server.metrics().items()})
        if self.text is not None and hasattr(self.text, "metrics"):
            m = self.text.metrics() if callable(self.text.metrics) else self.text.metrics
            out.update({f"text/{k}": v for k, v in dict(m).items() if isinstance(v, (int, float))})
        return out
