"""File-backed record sources beside ``Files`` / ``TokenFiles``: JSON lines, Parquet, and a Hub-style snapshot directory.

There is no network access at run time, so ``Hub`` resolves a dataset id to a *local* snapshot (the layout
``huggingface_hub`` leaves under its cache: ``datasets--<org>--<name>/snapshots/<rev>/``, or any directory given) and reads the
Parquet / JSON-lines files it finds there; a snapshot that is not present raises with the path that was searched.
Reference: the ``Hub`` / ``TFDS`` sources of src/dew/data/.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

from .dataset import Dataset


class JsonLines(Dataset):
    """One JSON object per line; records are loaded eagerly (line offsets could be indexed for larger files)."""

    def __init__(self, paths: Sequence[os.PathLike] | os.PathLike):
        paths = [paths] if isinstance(paths, (str, os.PathLike)) else list(paths)
        rows: List[Dict[str, Any]] = []
        for p in paths:
            with open(p) as f:
                rows += [json.loads(line) for line in f if line.strip()]
        super().__init__(rows)


class Parquet(Dataset):
    """Rows of one or more Parquet files (read with pyarrow, column subset optional)."""

    def __init__(self, paths: Sequence[os.PathLike] | os.PathLike, columns: Optional[Sequence[str]] = None):
        import pyarrow.parquet as pq
        paths = [paths] if isinstance(paths, (str, os.PathLike)) else list(paths)
        tables = [pq.read_table(str(p), columns=list(columns) if columns else None) for p in paths]
        rows: List[Dict[str, Any]] = []
        for t in tables:
            rows += t.to_pylist()
        super().__init__(rows)


class Hub(Dataset):
    """``Hub("org/name", split="train")``: the records of a locally available snapshot of a hub dataset."""

    def __init__(self, repo_id: str, split: str = "train", cache_dir: Optional[os.PathLike] = None, revision: Optional[str] = None,
                 columns: Optional[Sequence[str]] = None):
        root = self.snapshot(repo_id, cache_dir, revision)
        files = sorted(p for p in root.rglob("*") if p.is_file() and split in p.name and p.suffix in (".parquet", ".jsonl", ".json"))
        if not files:
            files = sorted(p for p in root.rglob("*") if p.is_file() and p.suffix in (".parquet", ".jsonl"))
        if not files:
            raise FileNotFoundError(f"{root} holds no parquet / jsonl files for split {split!r}")
        rows: List[Dict[str, Any]] = []
        for p in files:
            src = Parquet(p, columns) if p.suffix == ".parquet" else JsonLines(p)
            rows += [src._get(i) for i in range(len(src))]
        super().__init__(rows)

    @staticmethod
    def snapshot(repo_id: str, cache_dir: Optional[os.PathLike] = None, revision: Optional[str] = None) -> Path:
        direct = Path(repo_id)
        if direct.is_dir():
            return direct
        base = Path(cache_dir or os.environ.get("HF_DATASETS_CACHE") or os.environ.get("HF_HOME", Path.home() / ".cache" / "huggingface") )
        for hub in (base, base / "hub"):
            snaps = hub / ("datasets--" + repo_id.replace("/", "--")) / "snapshots"
            if snaps.is_dir():
                revs = sorted(p for p in snaps.iterdir() if p.is_dir())
                if revision:
                    revs = [p for p in revs if p.name.startswith(revision)]
                if revs:
                    return revs[-1]
        raise FileNotFoundError(f"no local snapshot of dataset {repo_id!r} under {base} (this process has no network access: "
                                "place the snapshot there or pass a directory)")


class Concatenate(Dataset):
    """Several map-style datasets read one after another as one (their own stages are not applied: concatenate sources, then chain)."""

    def __init__(self, parts: Sequence[Dataset]):
        sizes = [len(p) for p in parts]
        if any(p._length is None for p in parts):
            raise ValueError("only datasets of known length concatenate")
        super().__init__(None, length=sum(sizes))
        self._parts = list(parts)
        self._starts = [0]
        for n in sizes:
            self._starts.append(self._starts[-1] + n)

    def _get(self, i: int):
        import bisect
        j = bisect.bisect_right(self._starts, i) - 1
        return self._parts[j]._get(i - self._starts[j])


class TorchDataset(Dataset):
    """A map-style ``torch.utils.data.Dataset`` (``__len__`` / ``__getitem__``) read through the shared chain.  ``fields`` names the entries
    of a tuple sample (``("image", "label")``); a mapping sample is taken as it is."""

    def __init__(self, dataset, fields: Optional[Sequence[str]] = None):
        super().__init__(None, length=len(dataset))
        self._dataset, self._fields = dataset, tuple(fields) if fields else None

    def _get(self, i: int):
        sample = self._dataset[i]
        if isinstance(sample, dict):
            return sample
        if self._fields is None:
            raise TypeError("a tuple sample needs field names: TorchDataset(ds, fields=('image', 'label'))")
        if len(sample) != len(self._fields):
            raise ValueError(f"a sample holds {len(sample)} entries, {len(self._fields)} field names were given")
        return dict(zip(self._fields, sample))


class HFDataset(TorchDataset):
    """A Hugging Face ``datasets.Dataset`` (already loaded: this library fetches nothing) read as a store; ``columns`` keeps a subset."""

    def __init__(self, dataset, columns: Optional[Sequence[str]] = None):
        super().__init__(dataset)
        self._columns = tuple(columns) if columns else None

    def _get(self, i: int):
        row = dict(self._dataset[int(i)])
        return row if self._columns is None else {k: row[k] for k in self._columns}


class IteratorSource(Dataset):
    """Any re-creatable iterator read as a store: ``factory()`` returns a fresh iterator over the same records in the same order.  The
    position counts delivered rows; a restore reads the iterator again up to it."""

    def __init__(self, factory, length: Optional[int] = None):
        super().__init__(None, length=length)
        self._factory = factory

    def _rows(self, skip_rows: int = 0):
        while True:
            n = 0
            for record in self._factory():
                for row in self._through(record):
                    n += 1
                    if skip_rows:
                        skip_rows -= 1
                        continue
                    yield row
            if not self._repeat or n == 0:
                return
