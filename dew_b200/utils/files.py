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
    atomic_write_bytes(path, json.dumps(value, indent=1, sort_keys=True, default=str).encode())


def read_json(path: os.PathLike) -> Any:
    with open(path, "rb") as f:
        return json.loads(f.read())
