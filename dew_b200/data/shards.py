"""Tar shards of samples (the WebDataset convention): a sample is the consecutive members of a tar that share a basename, each
member a field named by its extension (``0001.jpg``, ``0001.txt``, ``0001.json``).  Shards are the unit of partitioning - rank r
of w reads shards r, r + w, ... - and of resumption: the position is (shard, sample within shard), so a resumed reader skips
whole shards without reading them.

``write_shards(samples, directory, samples_per_shard)``   writes ``shard-00000.tar`` ... and an ``index.json`` with counts
``TarShards(directory | paths)``                           a ``Dataset`` streaming the samples; ``.shuffle`` permutes shards per
                                                           epoch and samples inside a buffer

Reference: src/dew/data/shards.py, src/dew/data/storage.py (sharded storage, an index with per-shard counts, resumable reads).
"""
from __future__ import annotations

import io
import json
import os
import tarfile
from typing import Any, Dict, Iterable, Iterator, List, Mapping, Optional, Sequence

import numpy as np

from .dataset import DataPartition, Dataset, collate

INDEX = "index.json"


def _encode(value: Any) -> bytes:
    if isinstance(value, bytes):
        return value
    if isinstance(value, str):
        return value.encode("utf-8")
    if isinstance(value, np.ndarray):
        buf = io.BytesIO()
        np.save(buf, value, allow_pickle=False)
        return buf.getvalue()
    return json.dumps(value).encode("utf-8")


def _decode(ext: str, data: bytes) -> Any:
    if ext in ("txt", "text", "caption"):
        return data.decode("utf-8")
    if ext in ("json",):
        return json.loads(data)
    if ext in ("npy",):
        return np.load(io.BytesIO(data), allow_pickle=False)
    if ext in ("cls", "id"):
        return int(data.decode())
    return data                                                          # images and anything else stay bytes (decoded by a map stage)


def write_shards(samples: Iterable[Mapping[str, Any]], directory: str, samples_per_shard: int = 1000, prefix: str = "shard") -> Dict[str, Any]:
    """Each sample is a mapping field-extension -> value (``{"jpg": bytes, "txt": "a cat", "json": {...}}``), with an optional
    ``__key__``.  Returns the index written."""
    os.makedirs(directory, exist_ok=True)
    shards: List[Dict[str, Any]] = []
    tar = None
    count = total = 0

    def close():
        nonlocal tar
        if tar is not None:
            tar.close()
            os.replace(shards[-1]["path_tmp"], os.path.join(directory, shards[-1]["file"]))
            shards[-1].pop("path_tmp")
            shards[-1]["samples"] = count
            tar = None

    for sample in samples:
        if tar is None or count >= samples_per_shard:
            close()
            name = f"{prefix}-{len(shards):05d}.tar"
            shards.append({"file": name, "path_tmp": os.path.join(directory, name + ".tmp"), "samples": 0})
            tar = tarfile.open(shards[-1]["path_tmp"], "w")
            count = 0
        key = str(sample.get("__key__", f"{total:09d}"))
        for ext, value in sample.items():
            if ext == "__key__":
                continue
            data = _encode(value)
            info = tarfile.TarInfo(f"{key}.{ext}")
            info.size = len(data)
            tar.addfile(info, io.BytesIO(data))
        count += 1
        total += 1
    close()
    index = {"shards": shards, "samples": total}
    with open(os.path.join(directory, INDEX + ".tmp"), "w") as f:
        json.dump(index, f)
    os.replace(os.path.join(directory, INDEX + ".tmp"), os.path.join(directory, INDEX))
    return index


def read_shard(path: str) -> Iterator[Dict[str, Any]]:
    with tarfile.open(path, "r") as tar:
        current, key = {}, None
        for member in tar:
            if not member.isfile():
                continue
            base, _, ext = member.name.partition(".")
            if key is not None and base != key:
                yield {"__key__": key, **current}
                current = {}
            key = base
            current[ext] = _decode(ext.rsplit(".", 1)[-1], tar.extractfile(member).read())
        if key is not None:
            yield {"__key__": key, **current}


class TarShards(Dataset):
    def __init__(self, source, buffer: int = 256):
        if isinstance(source, (str, os.PathLike)):
            directory = str(source)
            with open(os.path.join(directory, INDEX)) as f:
                index = json.load(f)
            self._shards = [(os.path.join(directory, s["file"]), int(s["samples"])) for s in index["shards"]]
        else:
            self._shards = [(str(p), None) for p in source]
        self._buffer = buffer
        total = sum(n for _, n in self._shards) if all(n is not None for _, n in self._shards) else None
        super().__init__(records=None, length=total)
        self._shard_at = 0          # position: shards of this partition fully read, and samples read of the current one
        self._sample_at = 0

    def _my_shards(self, epoch: int) -> List[int]:
        order = np.arange(len(self._shards))
        if self._shuffle_seed is not None:
            order = np.random.default_rng((self._shuffle_seed, epoch)).permutation(len(self._shards))
        return [int(s) for s in order[self._partition.index::self._partition.count]]

    def _samples(self) -> Iterator[Any]:
        epoch = 0
        while True:
            mine = self._my_shards(epoch)
            for si in range(self._shard_at, len(mine)):
                path, _ = self._shards[mine[si]]
                for k, sample in enumerate(read_shard(path)):
                    if k < self._sample_at:
                        continue
                    self._sample_at = k + 1
                    for fn in self._maps:
                        sample = fn(sample)
                    yield sample
                self._shard_at, self._sample_at = si + 1, 0
            self._shard_at = 0
            epoch += 1
            if not self._repeat:
                return

    def _shuffled(self, gen: Iterator[Any]) -> Iterator[Any]:
        if self._shuffle_seed is None or self._buffer <= 1:
            yield from gen
            return
        rng = np.random.default_rng(self._shuffle_seed + 7919 * (self._partition.index + 1))
        held: List[Any] = []
        for s in gen:
            held.append(s)
            if len(held) >= self._buffer:
                yield held.pop(int(rng.integers(len(held))))
        while held:
            yield held.pop(int(rng.integers(len(held))))

    def __iter__(self) -> Iterator[Any]:
        gen = self._shuffled(self._samples())
        if self._batch is None:
            yield from gen
            return
        rows: List[Any] = []
        for r in gen:
            rows.append(r)
            if len(rows) == self._batch:
                yield collate(rows)
                rows = []
        if rows and not self._drop_last:
            yield collate(rows)

    def position(self) -> Dict[str, Any]:
        return {"shard": self._shard_at, "sample": self._sample_at, "partitions": self._partition.count}

    def restore(self, position: Mapping[str, Any]) -> None:
        if int(position.get("partitions", self._partition.count)) != self._partition.count:
            # the shards are dealt differently now: restart the epoch's shards (a shard is never half-counted twice within a run
            # of one partitioning; across a re-partitioning the epoch restarts)
            self._shard_at = self._sample_at = 0
            return
        self._shard_at, self._sample_at = int(position.get("shard", 0)), int(position.get("sample", 0))
