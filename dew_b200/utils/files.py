"""Atomic file writes and JSON helpers (reference: src/dew/_files.py)."""
from __future__ import annotations

import json
import os
import tempfile
from pathlib import Path
from typing import Any


def atomic_write_bytes(path: os.PathLike, data: bytes) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=str(path.parent), prefix=f".{path.name}.")
    try:
        with os.fdopen(fd, "wb") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def atomic_write_json(path: os.PathLike, value: Any) -> None:
    """Values JSON cannot express raise ``TypeError``: a tensor or an object written as its ``repr`` would read back as
    a string and lose the state it stood for."""
    atomic_write_bytes(path, json.dumps(value, indent=1, sort_keys=True, default=_plain).encode())


def _plain(v: Any) -> Any:
    # paths, sets / tuples and zero-dimensional numpy / torch numbers have one obvious JSON form; anything else is refused
    if isinstance(v, Path):
        return str(v)
    if isinstance(v, (set, frozenset, tuple)):
        return list(v)
    if hasattr(v, "item") and getattr(v, "ndim", None) == 0:
        return v.item()
    raise TypeError(f"{type(v).__name__} is not JSON serialisable: store tensors in the item's tensor file")


def read_json(path: os.PathLike) -> Any:
    with open(path, "rb") as f:
        return json.loads(f.read())
