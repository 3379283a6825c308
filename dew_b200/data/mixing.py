"""Weighted mixtures of datasets, curriculum phases and batch-size ramps.

``Mixture([(ds, weight), ...], seed)`` draws each next record from source ``i`` with probability ``w_i / sum w`` using a
counter-based stream keyed by ``(seed, draw index)``, so the interleaving is the same on any restart; its position (draws
made, per-source positions) is restorable.  ``PhasedStream`` switches sources at step boundaries; ``RampedStream`` grows
the batch size on a schedule.  Reference: src/dew/data (mixing, ``PhasedStream``, ``RampedStream``, ``Checkpointable``).
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Mapping, Sequence, Tuple

import numpy as np


class Mixture:
    def __init__(self, sources: Sequence[Tuple[Any, float]], seed: int = 0):
        self.sources = [s for s, _ in sources]
        w = np.asarray([float(x) for _, x in sources], dtype=np.float64)
        self.cum = np.cumsum(w / w.sum())
        self.seed, self.draws = seed, 0
        self.taken = [0] * len(self.sources)
        self._iters: List[Iterator] = []

    def _choice(self, n: int) -> int:
        u = np.random.default_rng([self.seed, n]).random()
        return int(np.searchsorted(self.cum, u, side="right").clip(0, len(self.sources) - 1))

    def __iter__(self):
        self._iters = [iter(s) for s in self.sources]
        # fast-forward each source to its restored position
        for it, n in zip(self._iters, self.taken):
            for _ in range(n):
                next(it)
        return self

    def __next__(self):
        i = self._choice(self.draws)
        try:
            rec = next(self._iters[i])
        except StopIteration:
            self._iters[i] = iter(self.sources[i])           # sources repeat independently
            self.taken[i] = 0
            rec = next(self._iters[i])
        self.draws += 1
        self.taken[i] += 1
        return rec

    def position(self) -> Dict[str, Any]:
        return {"draws": self.draws, "taken": list(self.taken)}

    def restore(self, position: Mapping[str, Any]) -> None:
        self.draws, self.taken = int(position["draws"]), [int(x) for x in position["taken"]]


class PhasedStream:
    """``phases = [(until_step, dataset), ...]``: batches come from the first phase whose bound exceeds the step."""

    def __init__(self, phases: Sequence[Tuple[int, Any]]):
        self.phases, self.step = list(phases), 0
        self._its: Dict[int, Iterator] = {}

    def __iter__(self):
        return self

    def __next__(self):
        for i, (until, ds) in enumerate(self.phases):
            if self.step < until or i == len(self.phases) - 1:
                if i not in self._its:
                    self._its[i] = iter(ds)
                self.step += 1
                return next(self._its[i])
        raise StopIteration

    def position(self):
        return {"step": self.step}

    def restore(self, position):
        self.step = int(position["step"])


class RampedStream:
    """Re-batches a stream of single records so that step ``s`` has ``schedule(s)`` rows (a batch-size ramp)."""

    def __init__(self, records, schedule, collate):
        self.records, self.schedule, self.collate, self.step = records, schedule, collate, 0

    def __iter__(self):
        self._it = iter(self.records)
        return self

    def __next__(self):
        n = int(self.schedule(self.step))
        rows = [next(self._it) for _ in range(n)]
        self.step += 1
        return self.collate(rows)
