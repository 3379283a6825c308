"""Sinks: write a dataset out as files that the sources read back (``TokenFiles`` shards, JSON lines).

``write_token_shards(rows of ids, directory, shard_tokens)`` packs documents into ``uint16`` / ``uint32`` binary shards
(``shard-00000.bin`` ...) with an ``index.json`` (dtype, counts, document boundaries), written atomically (temporary file
then rename) so a reader never sees half a shard.  ``write_jsonl`` does the same for records.

Reference: src/dew/data/sinks.py, src/dew/data/shards.py (sharded writers behind ``dew data export``).
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any, Iterable, List, Mapping, Sequence

import numpy as np


def _atomic(path: Path, data: bytes) -> None:
    tmp = path.with_name(path.name + ".tmp")
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def write_token_shards(documents: Iterable[Sequence[int]], directory, *, shard_tokens: int = 1 << 24, vocab_size: int = 1 << 16,
                       eos_id: int = None) -> dict:
    """Returns the index (also written to ``index.json``): ``{"dtype", "shards": [{"file", "tokens", "documents": [lengths]}]}``."""
    out = Path(directory)
    out.mkdir(parents=True, exist_ok=True)
    dtype = np.uint16 if vocab_size <= (1 << 16) else np.uint32
    shards: List[dict] = []
    cur: List[np.ndarray] = []
    lens: List[int] = []
    held = 0

    def flush():
        nonlocal cur, lens, held
        if not cur:
            return
        name = f"shard-{len(shards):05d}.bin"
        _atomic(out / name, np.concatenate(cur).astype(dtype).tobytes())
        shards.append({"file": name, "tokens": held, "documents": lens})
        cur, lens, held = [], [], 0

    for doc in documents:
        ids = np.asarray(list(doc) + ([eos_id] if eos_id is not None else []), dtype=np.int64)
        if ids.size and (ids.min() < 0 or ids.max() >= (1 << (16 if dtype == np.uint16 else 32))):
            raise ValueError("a token id does not fit the shard's dtype")
        if held and held + ids.size > shard_tokens:
            flush()
        cur.append(ids)
        lens.append(int(ids.size))
        held += int(ids.size)
    flush()
    index = {"dtype": np.dtype(dtype).name, "shards": shards, "tokens": sum(s["tokens"] for s in shards)}
    _atomic(out / "index.json", json.dumps(index).encode())
    return index


def read_token_shards(directory) -> Iterable[np.ndarray]:
    """The documents back, in order (one array of ids per document)."""
    d = Path(directory)
    index = json.loads((d / "index.json").read_text())
    for s in index["shards"]:
        flat = np.fromfile(d / s["file"], dtype=np.dtype(index["dtype"]))
        at = 0
        for n in s["documents"]:
            yield flat[at:at + n].astype(np.int64)
            at += n


def write_jsonl(records: Iterable[Mapping[str, Any]], path) -> int:
    lines = [json.dumps(r, ensure_ascii=False) for r in records]
    _atomic(Path(path), ("\n".join(lines) + ("\n" if lines else "")).encode())
    return len(lines)
