"""A stage's records run on a pool of its own, several at once, delivered in the order they were read.  ``OrderedPool(fn, workers,
depth)`` wraps a slow per-record function (a fetch, a decode): up to ``depth`` records are in flight on ``workers`` threads, results come
out in input order, an exception surfaces at the record that raised it, and ``position`` counts delivered records so a restore reads the
stream again from there (``restore(n)`` skips the first ``n`` inputs without running ``fn`` on them).

Reference: src/dew/data/concurrent.py (``Pool``; a fetch's threads).
"""
from __future__ import annotations

import collections
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Callable, Iterable, Iterator


class OrderedPool:
    def __init__(self, fn: Callable[[Any], Any], workers: int = 8, depth: int = 0):
        if workers < 1:
            raise ValueError("a pool runs on at least one worker")
        self.fn, self.workers, self.depth = fn, workers, depth or 2 * workers
        self.position = 0
        self._skip = 0

    def restore(self, position: int) -> None:
        self._skip = self.position = int(position)

    def __call__(self, stream: Iterable[Any]) -> Iterator[Any]:
        it = iter(stream)
        for _ in range(self._skip):                              # delivered before the restore: read past, do not run
            if next(it, _END) is _END:
                return
        self._skip = 0
        flight: "collections.deque" = collections.deque()
        with ThreadPoolExecutor(max_workers=self.workers) as pool:
            try:
                for record in it:
                    flight.append(pool.submit(self.fn, record))
                    if len(flight) >= self.depth:
                        out = flight.popleft().result()
                        self.position += 1
                        yield out
                while flight:
                    out = flight.popleft().result()
                    self.position += 1
                    yield out
            finally:
                for f in flight:
                    f.cancel()


_END = object()
