"""Orders of a streamed read.  ``locality_order``: visit the physical shards in a shuffled order and, inside a sliding window of a few
shards, interleave their records at random - a shuffle whose reads stay sequential per shard and that never materialises a permutation
of the records.  ``WindowShuffle``: a streamed shuffle in fixed windows of the stream - window ``i`` is permuted by ``(seed, i)`` alone,
so a restored position (a count of delivered records) finds its place by reading one window.  ``skipping``: an index order past the
places an earlier phase already trained on.

Reference: src/dew/data/ordering.py (locality order, ``WindowShuffle``, ``Skipping``).
"""
from __future__ import annotations

from typing import Any, Iterable, Iterator, List, Sequence, Set, Tuple

import numpy as np


def locality_order(shard_sizes: Sequence[int], seed: int = 0, epoch: int = 0, open_shards: int = 4) -> Iterator[Tuple[int, int]]:
    """``(shard, record)`` pairs covering every record once.  At most ``open_shards`` shards are read at a time, each front to back; the
    next record comes from one of the open shards, drawn in proportion to what each has left."""
    rng = np.random.default_rng((seed, epoch))
    pending = list(rng.permutation(len(shard_sizes)))
    open_: List[List[int]] = []                                # [shard, next record]
    while pending or open_:
        while pending and len(open_) < open_shards:
            s = int(pending.pop(0))
            if shard_sizes[s] > 0:
                open_.append([s, 0])
        if not open_:
            return
        left = np.array([shard_sizes[s] - at for s, at in open_], dtype=np.float64)
        j = int(rng.choice(len(open_), p=left / left.sum()))
        s, at = open_[j]
        yield s, at
        open_[j][1] += 1
        if open_[j][1] >= shard_sizes[s]:
            open_.pop(j)


class WindowShuffle:
    """``WindowShuffle(window, seed)(stream)`` yields the stream's records shuffled inside consecutive windows of ``window`` records.
    ``position`` counts delivered records; ``restore(position)`` makes the next iteration skip the windows before it without keeping their
    records and drop the delivered part of the window it falls in."""

    def __init__(self, window: int, seed: int = 0):
        if window < 1:
            raise ValueError("a shuffle window holds at least one record")
        self.window, self.seed, self.position = window, seed, 0

    def restore(self, position: int) -> None:
        self.position = int(position)

    def __call__(self, stream: Iterable[Any]) -> Iterator[Any]:
        skip_windows, within = divmod(self.position, self.window)
        buf: List[Any] = []
        w = 0
        for k, record in enumerate(stream):
            w = k // self.window
            if w < skip_windows:
                continue
            buf.append(record)
            if len(buf) == self.window:
                yield from self._emit(buf, w, within if w == skip_windows else 0)
                buf = []
        if buf:
            yield from self._emit(buf, w, within if w == skip_windows else 0)

    def _emit(self, buf: List[Any], w: int, drop: int) -> Iterator[Any]:
        order = np.random.default_rng((self.seed, w)).permutation(len(buf))
        for j, i in enumerate(order):
            if j < drop:
                continue
            self.position = w * self.window + j + 1
            yield buf[int(i)]


def skipping(order: Iterable[int], seen: Set[int]) -> Iterator[int]:
    """The indices of ``order`` that ``seen`` does not hold: a later phase's order past what an earlier one trained on."""
    return (i for i in order if i not in seen)
