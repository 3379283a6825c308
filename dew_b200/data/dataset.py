"""Data pipeline: chainable sources -> transforms -> batches, partitioned across data-parallel ranks, with a
checkpointable position.

Parity (capabilities): src/dew/data/dataset.py (``Loader``, ``DataPartition``, ``Checkpointable``), sources
``Memory / Files / TokenFiles``, ``.shuffle(seed).repeat().pipe(preset, ...).workers(n)``; position save / restore for
resume (``data_resume``), elastic re-partitioning (tests/test_data_elastic.py in the reference).
"""
from __future__ import annotations

import glob
import os
import queue
import threading
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Iterator, List, Mapping, Optional, Sequence

import numpy as np
import torch


@dataclass(frozen=True)
class DataPartition:
    """This process's share of the data: ``index`` of ``count`` partitions."""
    index: int = 0
    count: int = 1


def collate(rows: Sequence[Mapping[str, Any]]) -> Dict[str, torch.Tensor]:
    out = {}
    for k in rows[0]:
        vals = [r[k] for r in rows]
        if isinstance(vals[0], torch.Tensor):
            out[k] = torch.stack(vals)
        elif isinstance(vals[0], np.ndarray):
            out[k] = torch.from_numpy(np.stack(vals))
        elif isinstance(vals[0], (int, float, bool, np.integer, np.floating)):
            out[k] = torch.tensor(vals)
        else:
            out[k] = vals
    return out


class Dataset:
    """A lazily-evaluated chain.  Each stage wraps an iterator factory ``make(partition, epoch_seed, skip)``."""

    def __init__(self, records: Optional[Sequence[Any]] = None, length: Optional[int] = None):
        self._records = records
        self._length = length if length is not None else (len(records) if records is not None else None)
        self._shuffle_seed: Optional[int] = None
        self._repeat = False
        self._maps: List[Callable] = []
        self._batch: Optional[int] = None
        self._drop_last = True
        self._workers = 0
        self._partition = DataPartition()
        self._consumed = 0          # batches handed out (the checkpointable position)
        self.batch: Optional[int] = None
        self.seq_len: Optional[int] = None

    # ---- chain
    def _copy(self) -> "Dataset":
        import copy
        c = copy.copy(self)
        c._maps = list(self._maps)
        return c

    def shuffle(self, seed: int = 0) -> "Dataset":
        c = self._copy(); c._shuffle_seed = seed; return c

    def repeat(self) -> "Dataset":
        c = self._copy(); c._repeat = True; return c

    def map(self, fn: Callable) -> "Dataset":
        c = self._copy(); c._maps.append(fn); return c

    def filter(self, keep: Callable[[Any], bool]) -> "Dataset":
        """Rows for which ``keep(row)`` is false are dropped.  (After a stage that changes the number of rows, a restored position is found by
        reading the epoch again up to it: exact, and as slow as the rows it skips.)"""
        c = self._copy(); c._maps.append(_Stage("filter", keep)); return c

    def flat_map(self, fn: Callable[[Any], Iterable[Any]]) -> "Dataset":
        """Every row becomes the rows ``fn(row)`` yields (none, one or several): over-length splitting, windows over a document."""
        c = self._copy(); c._maps.append(_Stage("flat", fn)); return c

    def batched(self, batch: int, drop_last: bool = True) -> "Dataset":
        c = self._copy(); c._batch = batch; c.batch = batch; c._drop_last = drop_last; return c

    def pipe(self, preset: Callable, *args, **kwargs) -> "Dataset":
        return preset(self, *args, **kwargs)

    def workers(self, n: int) -> "Dataset":
        c = self._copy(); c._workers = n; return c

    def partition(self, part: DataPartition) -> "Dataset":
        c = self._copy(); c._partition = part; return c

    # ---- records
    def _get(self, i: int):
        return self._records[i]

    def __len__(self) -> int:
        return self._length or 0

    @property
    def steps_per_epoch(self) -> Optional[int]:
        if self._length is None or self._batch is None:
            return None
        return (self._length // self._partition.count) // self._batch

    def _order(self, epoch: int) -> np.ndarray:
        n = self._length
        idx = np.arange(n)
        if self._shuffle_seed is not None:
            idx = np.random.default_rng((self._shuffle_seed, epoch)).permutation(n)
        per = n // self._partition.count if self._partition.count > 1 else n
        lo = self._partition.index * per
        return idx[lo:lo + per]

    def _through(self, row, stage: int = 0) -> Iterator[Any]:
        """``row`` through the stages from ``stage`` on: zero, one or several rows."""
        for j in range(stage, len(self._maps)):
            fn = self._maps[j]
            if isinstance(fn, _Stage):
                if fn.kind == "filter":
                    if not fn.fn(row):
                        return
                    continue
                for out in fn.fn(row):
                    yield from self._through(out, j + 1)
                return
            row = fn(row)
        yield row

    def _rows(self, skip_rows: int = 0) -> Iterator[Any]:
        if any(isinstance(fn, _Stage) for fn in self._maps):
            # the position counts delivered rows, which no longer map to source rows: read from the start and drop what was delivered
            epoch, dropped = 0, 0
            while True:
                for i in self._order(epoch):
                    for row in self._through(self._get(int(i))):
                        if dropped < skip_rows:
                            dropped += 1
                            continue
                        yield row
                epoch += 1
                if not self._repeat:
                    return
        epoch = 0
        per_epoch = len(self._order(0))
        if per_epoch:
            epoch, skip_rows = divmod(skip_rows, per_epoch) if self._repeat else (0, skip_rows)
        while True:
            for i in self._order(epoch)[skip_rows:]:
                row = self._get(int(i))
                for fn in self._maps:
                    row = fn(row)
                yield row
            skip_rows = 0
            epoch += 1
            if not self._repeat:
                return

    def __iter__(self) -> Iterator[Any]:
        start = self._consumed
        if self._batch is None:
            src = self._rows(start)
            gen = src
        else:
            def batches():
                rows = []
                for r in self._rows(start * self._batch):
                    rows.append(r)
                    if len(rows) == self._batch:
                        yield collate(rows)
                        rows = []
                if rows and not self._drop_last:
                    yield collate(rows)
            gen = batches()
        if self._workers > 0:
            gen = _prefetch(gen, depth=2 * self._workers)
        for item in gen:
            self._consumed += 1
            yield item

    # ---- checkpointable position
    def position(self) -> Dict[str, Any]:
        return {"consumed": int(self._consumed), "partitions": int(self._partition.count)}

    def restore(self, position: Mapping[str, Any]) -> None:
        consumed = int(position.get("consumed", 0))
        old = int(position.get("partitions", self._partition.count))
        # elastic: the same global number of batches, re-split over the new partition count
        self._consumed = consumed * old // max(1, self._partition.count)


class _Stage:
    """A stage that changes the number of rows: ``filter`` or ``flat``."""
    __slots__ = ("kind", "fn")

    def __init__(self, kind: str, fn: Callable):
        self.kind, self.fn = kind, fn


def _prefetch(gen: Iterable[Any], depth: int = 4) -> Iterator[Any]:
    q: "queue.Queue" = queue.Queue(maxsize=depth)
    END = object()

    def work():
        try:
            for item in gen:
                q.put(item)
            q.put(END)
        except BaseException as e:
            q.put(e)
    threading.Thread(target=work, daemon=True).start()
    while True:
        item = q.get()
        if item is END:
            return
        if isinstance(item, BaseException):
            raise item
        yield item


class Memory(Dataset):
    """Records held in memory (a list of mappings, or a mapping of equal-length arrays)."""

    def __init__(self, records):
        if isinstance(records, Mapping):
            n = len(next(iter(records.values())))
            self._columns = records
            super().__init__(None, n)
        else:
            self._columns = None
            super().__init__(list(records))

    def _get(self, i):
        if self._columns is not None:
            return {k: v[i] for k, v in self._columns.items()}
        return self._records[i]


class Files(Dataset):
    """One record per file matching a glob; ``read`` turns a path into a record."""

    def __init__(self, pattern: str, read: Callable[[str], Any] = lambda p: {"path": p}):
        self.paths = sorted(glob.glob(pattern, recursive=True))
        self.read = read
        super().__init__(None, len(self.paths))

    def _get(self, i):
        return self.read(self.paths[i])


class TokenFiles(Dataset):
    """Flat binary token files (uint16 / uint32 / int32) memory-mapped; records are fixed windows of tokens."""

    def __init__(self, path: str, dtype: str = "uint16", window: Optional[int] = None):
        paths = sorted(glob.glob(path)) if any(c in path for c in "*?[") else [path]
        self.arrays = [np.memmap(p, dtype=np.dtype(dtype), mode="r") for p in paths]
        self.window = window
        self.total = sum(len(a) for a in self.arrays)
        super().__init__(None, self.total if window is None else self.total // window)

    def set_window(self, window: int) -> "TokenFiles":
        c = self._copy(); c.window = window; c._length = self.total // window; return c

    def _get(self, i):
        off = i * self.window
        for a in self.arrays:
            if off + self.window <= len(a):
                return {"tokens": torch.from_numpy(np.asarray(a[off:off + self.window]).astype(np.int64))}
            off -= (len(a) // self.window) * self.window
        raise IndexError(i)


class Loader:
    """Wraps user callables: ``train(partition) -> iterator of batches`` (and ``val``)."""

    def __init__(self, train: Callable[[DataPartition], Iterable], val: Optional[Callable] = None,
                 records: Optional[int] = None, batch: Optional[int] = None, seq_len: Optional[int] = None,
                 partition: DataPartition = DataPartition()):
        self._train, self._val = train, val
        self.records, self.batch, self.seq_len = records, batch, seq_len
        self._partition = partition
        self._consumed = 0

    @property
    def steps_per_epoch(self):
        if self.records is None or self.batch is None:
            return None
        return self.records // (self.batch * self._partition.count)

    def train(self):
        return self

    def __iter__(self):
        skip = self._consumed
        for i, b in enumerate(self._train(self._partition)):
            if i < skip:
                continue
            self._consumed += 1
            yield b

    def val(self):
        return iter(self._val(self._partition)) if self._val is not None else iter(())

    def position(self):
        return {"consumed": int(self._consumed), "partitions": int(self._partition.count)}

    def restore(self, position):
        self._consumed = int(position.get("consumed", 0))
