"""Held-out splits that do not depend on order, count or shuffling: a row belongs to the holdout when a hash of its key falls
under the holdout's share, so adding rows, re-sharding or resuming never moves a row across the split, and two datasets that
share rows (a dedup, a re-crawl) hold the same ones out.

``Holdout(fraction, salt)``           ``.is_held(key)``, ``.split(dataset)`` -> (train, held)
``group_key``                         rows that must stay together (a document's chunks, a user's sessions) share a group key
``stratified_counts``                 how a split fell per class, to check it

Reference: src/dew/data/holdout.py (hash-keyed holdouts, grouped rows, the selection recorded with the run).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

from .dataset import Dataset


def unit_hash(key: Any, salt: str = "") -> float:
    """A number in [0, 1) from ``key``, uniform over keys, fixed across processes and Python versions."""
    h = hashlib.blake2b(f"{salt}\x1f{key}".encode(), digest_size=8).digest()
    return int.from_bytes(h, "big") / 2.0 ** 64


@dataclass(frozen=True)
class Holdout:
    fraction: float = 0.01
    salt: str = "holdout"
    key: Optional[str] = None            # the row field to hash (default: "key" / "id" / "path" / "text", whichever exists first)

    def __post_init__(self):
        if not 0.0 <= self.fraction <= 1.0:
            raise ValueError("a holdout's share lies in [0, 1]")

    def key_of(self, row: Any) -> Any:
        if not isinstance(row, Mapping):
            return row
        if self.key is not None:
            return row[self.key]
        for name in ("group", "key", "id", "path", "text", "prompt"):
            if name in row:
                return row[name]
        raise KeyError("the row names no key to hold out by: give Holdout(key=...)")

    def is_held(self, key: Any) -> bool:
        return unit_hash(key, self.salt) < self.fraction

    def split(self, dataset: Dataset) -> Tuple[Dataset, Dataset]:
        """Two datasets over ``dataset``'s records (read once to index them): the training rows and the held-out ones."""
        n = len(dataset)
        held = [i for i in range(n) if self.is_held(self.key_of(dataset._get(i)))]
        held_set = set(held)
        train = [i for i in range(n) if i not in held_set]
        return _Subset(dataset, train), _Subset(dataset, held)

    def record(self) -> Dict[str, Any]:
        return {"fraction": self.fraction, "salt": self.salt, "key": self.key}


class _Subset(Dataset):
    def __init__(self, base: Dataset, indices):
        self._base, self._indices = base, list(indices)
        super().__init__(records=None, length=len(self._indices))
        self._maps = list(base._maps)

    def _get(self, i: int):
        return self._base._get(self._indices[i])


def stratified_counts(dataset: Dataset, label: str) -> Dict[Any, int]:
    out: Dict[Any, int] = {}
    for i in range(len(dataset)):
        v = dataset._get(i)[label]
        out[v] = out.get(v, 0) + 1
    return out
