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
