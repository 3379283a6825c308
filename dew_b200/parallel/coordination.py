"""Host-side coordination: agreements before collective phases, fail-fast publication of errors, pool teardown.

Parity: src/dew/_coordination.py (``collective_host`` :139-202, ``agreed`` :280, ``agreed_same`` :338, ``PeerFailure``
:377, ``publish_failure`` :541, ``end_pool_on_failure`` :595-655, ``agreement_patience``).  The KV store is
``torch.distributed.TCPStore`` (or any object with ``set / get / add / wait``); nothing here touches a GPU, so a rank
that raised can tell its peers before they enter a collective and hang.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
import threading
import time
import traceback
from dataclasses import dataclass
from typing import Any, Callable, List, Optional

FAILURE_GRACE_SECONDS = 60.0
FAILURE_KEY = "dewb/failure"


class PeerFailure(RuntimeError):
    """Another process of the pool published a failure."""

    def __init__(self, rank: int, message: str):
        super().__init__(f"process {rank} failed: {message}")
        self.rank, self.message = rank, message


class AgreementTimeout(TimeoutError):
    pass


@dataclass
class Pool:
    """This process's view of the pool: a store, its rank and the process count."""
    store: Any
    rank: int
    count: int
    patience: float = 24 * 3600.0       # how long an agreement may wait for slow peers
    _round: int = 0

    # ------------------------------------------------------------------ failure publication
    def publish_failure(self, exc: BaseException) -> None:
        msg = json.dumps({"rank": self.rank, "error": f"{type(exc).__name__}: {exc}"})
        try:
            self.store.set(FAILURE_KEY, msg)
        except Exception:
            pass

    def failure(self) -> Optional[PeerFailure]:
        try:
            if hasattr(self.store, "check") and not self.store.check([FAILURE_KEY]):
                return None
            raw = self.store.get(FAILURE_KEY)
        except Exception:
            return None
        if not raw:
            return None
        d = json.loads(raw.decode() if isinstance(raw, bytes) else raw)
        return PeerFailure(int(d["rank"]), d["error"]) if int(d["rank"]) != self.rank else None

    # ------------------------------------------------------------------ gathers and agreements
    def gather(self, phase: str, value: Any, poll: float = 0.02) -> List[Any]:
        """Every process contributes a JSON value; everyone receives the list in rank order. Raises ``PeerFailure`` if a
        peer published a failure while waiting, ``AgreementTimeout`` after ``patience``."""
        self._round += 1
        base = f"dewb/gather/{phase}/{self._round}"
        self.store.set(f"{base}/{self.rank}", json.dumps(value))
        out: List[Any] = [None] * self.count
        deadline = time.monotonic() + self.patience
        pending = set(range(self.count))
        while pending:
            f = self.failure()
            if f is not None:
                raise f
            for r in list(pending):
                key = f"{base}/{r}"
                ready = self.store.check([key]) if hasattr(self.store, "check") else True
                if ready:
                    raw = self.store.get(key)
                    out[r] = json.loads(raw.decode() if isinstance(raw, bytes) else raw)
                    pending.discard(r)
            if pending:
                if time.monotonic() > deadline:
                    raise AgreementTimeout(f"{phase}: processes {sorted(pending)} did not arrive within {self.patience}s")
                time.sleep(poll)
        return out

    def agreed(self, phase: str, decide: Callable[[], Any]) -> Any:
        """Rank 0 decides, everyone adopts its decision (e.g. which step to checkpoint at)."""
        mine = decide() if self.rank == 0 else None
        return self.gather(phase, mine)[0]

    def agreed_next(self, phase: str, proposal: int) -> int:
        """The earliest value every process can reach: the maximum of the proposals (an agreed future step)."""
        return max(self.gather(phase, int(proposal)))

    def agreed_same(self, phase: str, value: Any) -> Any:
        """All processes must hold the same value (compared by sha256 digest); raises naming the ranks that differ."""
        digest = hashlib.sha256(json.dumps(value, sort_keys=True, default=str).encode()).hexdigest()
        all_digests = self.gather(phase, digest)
        if len(set(all_digests)) != 1:
            odd = [r for r, d in enumerate(all_digests) if d != all_digests[0]]
            raise RuntimeError(f"{phase}: processes {odd} disagree with process 0")
        return value

    def barrier(self, phase: str = "barrier") -> None:
        self.gather(phase, 1)


def end_pool_on_failure(pool: Pool, grace: float = FAILURE_GRACE_SECONDS, poll: float = 0.5,
                        on_failure: Optional[Callable[[PeerFailure], None]] = None) -> threading.Thread:
    """Install an excepthook that publishes this process's failure and exits at once, and start a watch thread that ends
    this process within ``grace`` seconds of a peer's failure (so nobody hangs in a collective)."""
    previous = sys.excepthook

    def hook(kind, value, tb):
        pool.publish_failure(value)
        previous(kind, value, tb)
        os._exit(1)
    sys.excepthook = hook

    def watch():
        while True:
            f = pool.failure()
            if f is not None:
                if on_failure is not None:
                    on_failure(f)
                    return
                print(f"[dew_b200] {f}; ending this process", file=sys.stderr, flush=True)
                time.sleep(min(grace, 1.0))
                os._exit(1)
            time.sleep(poll)
    t = threading.Thread(target=watch, name="dewb-failure-watch", daemon=True)
    t.start()
    return t


class DictStore:
    """An in-process store with the TCPStore surface (tests, single process)."""

    def __init__(self):
        self._d, self._lock = {}, threading.Lock()

    def set(self, k, v):
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        with self._lock:
            return self._d.get(k, b"")

    def check(self, keys):
        with self._lock:
            return all(k in self._d for k in keys)

    def add(self, k, n):
        with self._lock:
            v = int(self._d.get(k, b"0")) + n
            self._d[k] = str(v).encode()
            return v
