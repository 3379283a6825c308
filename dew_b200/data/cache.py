"""On-disk cache of a prepared dataset: the records a pipeline produces (tokenised, packed, transformed) are written once
under a key derived from what produced them, and later runs memory-map them instead of recomputing.

    cached = Cached(lambda: presets.lm(raw, tok, seq_len=2048, batch=8), directory, key=("lm", tok.name, 2048))

The cache entry is a directory ``<directory>/<digest>/`` holding one ``.npy`` file per field (memory-mapped on read), a
``meta.json`` with the field names, shapes and the key, and a ``COMPLETE`` marker written last; an entry without the marker
(a run cut short) is rebuilt.  Reference: the dataset cache of src/dew/data/ (``cache``) and its atomic writes
(src/dew/_files.py).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from pathlib import Path
from typing import Any, Callable, Dict, Mapping, Sequence

import numpy as np
import torch

from .dataset import Dataset, Memory


def digest(key: Any) -> str:
    return hashlib.sha256(json.dumps(key, sort_keys=True, default=str).encode()).hexdigest()[:24]


def write_entry(directory: Path, fields: Mapping[str, np.ndarray], key: Any) -> None:
    tmp = directory.with_name(directory.name + f".partial{os.getpid()}")
    if tmp.exists():
        shutil.rmtree(tmp)
    tmp.mkdir(parents=True)
    for name, arr in fields.items():
        np.save(tmp / f"{name}.npy", np.ascontiguousarray(arr))
    (tmp / "meta.json").write_text(json.dumps({"key": key, "fields": {k: [list(v.shape), str(v.dtype)] for k, v in fields.items()}},
                                              default=str, indent=1))
    (tmp / "COMPLETE").write_text("ok")
    if directory.exists():
        shutil.rmtree(directory)
    os.replace(tmp, directory)


def read_entry(directory: Path) -> Dict[str, np.ndarray]:
    meta = json.loads((directory / "meta.json").read_text())
    return {name: np.load(directory / f"{name}.npy", mmap_mode="r") for name in meta["fields"]}


class Cached:
    """``Cached(build, directory, key)``: ``.dataset()`` returns a ``Memory`` dataset over the cached fields, building (and
    writing) them with ``build()`` on the first use.  ``build`` returns a ``Dataset`` of records (mappings of equal-shaped
    arrays) or a mapping of stacked arrays."""

    def __init__(self, build: Callable[[], Any], directory: os.PathLike, key: Any):
        self.build, self.root, self.key = build, Path(directory), key
        self.path = self.root / digest(key)

    def ready(self) -> bool:
        return (self.path / "COMPLETE").exists()

    def fields(self) -> Dict[str, np.ndarray]:
        if not self.ready():
            made = self.build()
            if isinstance(made, Mapping):
                fields = {k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in made.items() if k != "fill"}
            else:
                rows = [made._get(i) for i in range(len(made))]
                fields = {k: np.stack([np.asarray(r[k]) for r in rows]) for k in rows[0]}
            self.root.mkdir(parents=True, exist_ok=True)
            write_entry(self.path, fields, self.key)
        return read_entry(self.path)

    def dataset(self) -> Dataset:
        return Memory({k: torch.from_numpy(np.asarray(v)) for k, v in self.fields().items()})
