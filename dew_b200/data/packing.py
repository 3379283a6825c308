"""Sequence packing: documents of uneven length into fixed windows with segment ids and per-document positions.

Two packers:

``pack_whole``   never splits a document: best-fit-decreasing bin packing of whole documents into windows of ``seq_len + 1``
                 tokens (documents longer than a window are truncated, or split with ``split_long``); padding fills the rest.
                 This is the layout packed-document attention wants (segment ids non-decreasing along a row, 0 = padding).
``Packer``       streaming: documents arrive one by one, rows leave as soon as ``open_rows`` windows are in flight and the
                 fullest cannot take the next document; bounded memory for corpora that do not fit in RAM.

Every row carries ``tokens``, ``segments`` (1, 2, ... per document within the row; 0 for padding) and ``positions`` (the
token's index inside its own document, so rotary embeddings restart at every document).

Reference: packing of the LM data presets (src/dew/data/, ``presets.lm(pack=True)``), ``segments`` as the attention mask
source (src/dew/objectives/lm/objective.py ``_targets``).
"""
from __future__ import annotations

from typing import Dict, Iterable, Iterator, List, Optional, Sequence

import numpy as np


def _row(docs: Sequence[Sequence[int]], length: int, pad_id: int) -> Dict[str, np.ndarray]:
    tokens = np.full(length, pad_id, dtype=np.int64)
    segments = np.zeros(length, dtype=np.int32)
    positions = np.zeros(length, dtype=np.int32)
    at = 0
    for s, d in enumerate(docs, start=1):
        n = len(d)
        tokens[at:at + n] = d
        segments[at:at + n] = s
        positions[at:at + n] = np.arange(n)
        at += n
    return {"tokens": tokens, "segments": segments, "positions": positions}


def pack_whole(docs: Sequence[Sequence[int]], seq_len: int, pad_id: int = 0, eos_id: Optional[int] = None,
               split_long: bool = False) -> Dict[str, np.ndarray]:
    """Best-fit-decreasing packing of whole documents.  Returns stacked ``tokens / segments / positions [rows, seq_len + 1]``
    and ``fill`` (the fraction of non-padding tokens)."""
    L = seq_len + 1
    pieces: List[List[int]] = []
    for d in docs:
        d = list(d) + ([eos_id] if eos_id is not None else [])
        if len(d) > L:
            if split_long:
                pieces += [d[i:i + L] for i in range(0, len(d), L)]
            else:
                pieces.append(d[:L])
        elif d:
            pieces.append(d)
    order = sorted(range(len(pieces)), key=lambda i: -len(pieces[i]))
    bins: List[List[int]] = []          # indices of pieces per row
    space: List[int] = []
    for i in order:
        n = len(pieces[i])
        best, best_left = -1, L + 1
        for b, s in enumerate(space):   # the fullest row that still takes the piece
            if n <= s and s - n < best_left:
                best, best_left = b, s - n
        if best < 0:
            bins.append([i]); space.append(L - n)
        else:
            bins[best].append(i); space[best] -= n
    rows = [_row([pieces[i] for i in sorted(b)], L, pad_id) for b in bins]       # original order inside a row
    used = sum(len(p) for p in pieces)
    out = {k: np.stack([r[k] for r in rows]) if rows else np.zeros((0, L), dtype=np.int64) for k in ("tokens", "segments", "positions")}
    out["fill"] = used / max(1, len(rows) * L)
    return out


class Packer:
    """Streaming packer: ``add(document)`` yields finished rows; ``flush()`` yields what is still open."""

    def __init__(self, seq_len: int, pad_id: int = 0, eos_id: Optional[int] = None, open_rows: int = 16):
        self.L, self.pad_id, self.eos_id, self.open_rows = seq_len + 1, pad_id, eos_id, open_rows
        self._open: List[List[List[int]]] = []
        self._space: List[int] = []

    def add(self, doc: Sequence[int]) -> Iterator[Dict[str, np.ndarray]]:
        d = list(doc) + ([self.eos_id] if self.eos_id is not None else [])
        d = d[: self.L]
        if not d:
            return
        n = len(d)
        best, best_left = -1, self.L + 1
        for b, s in enumerate(self._space):
            if n <= s and s - n < best_left:
                best, best_left = b, s - n
        if best >= 0:
            self._open[best].append(d); self._space[best] -= n
            if self._space[best] == 0:
                yield self._close(best)
            return
        if len(self._open) >= self.open_rows:          # no room anywhere: the fullest open row leaves
            yield self._close(min(range(len(self._space)), key=self._space.__getitem__))
        self._open.append([d]); self._space.append(self.L - n)

    def _close(self, b: int) -> Dict[str, np.ndarray]:
        docs = self._open.pop(b)
        self._space.pop(b)
        return _row(docs, self.L, self.pad_id)

    def flush(self) -> Iterator[Dict[str, np.ndarray]]:
        while self._open:
            yield self._close(0)

    def pack(self, docs: Iterable[Sequence[int]]) -> Iterator[Dict[str, np.ndarray]]:
        for d in docs:
            yield from self.add(d)
        yield from self.flush()
