"""Record steps any chain takes.  Generic: field selection, renaming, formatting, predicates.  Token records: what to do with a record
longer than the model reads (truncate it, drop it, split it, or refuse), fixed-length checks, the count of targets a row trains on, and
overlapping causal windows - consecutive windows share their boundary token, so every token of a document is predicted exactly once
(disjoint windows would never predict each window's first token from its predecessor).

``dataset.map(select("tokens"))``, ``dataset.flat_map(over_length(2048, "split"))``, ``dataset.flat_map(causal_windows(2048))``.

Reference: src/dew/data/steps/generic.py, steps/text.py, steps/windows.py.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterable, Iterator, Mapping, Optional, Sequence

import numpy as np


def select(*fields: str) -> Callable[[Mapping[str, Any]], Dict[str, Any]]:
    def step(row):
        missing = [f for f in fields if f not in row]
        if missing:
            raise KeyError(f"record holds no {missing}; it holds {sorted(row)}")
        return {f: row[f] for f in fields}
    return step


def rename(**names: str) -> Callable[[Mapping[str, Any]], Dict[str, Any]]:
    """``rename(text="content")``: the field ``content`` becomes ``text``."""
    back = {old: new for new, old in names.items()}

    def step(row):
        return {back.get(k, k): v for k, v in row.items()}
    return step


def formatted(template: str, into: str = "text") -> Callable[[Mapping[str, Any]], Dict[str, Any]]:
    """``formatted("Q: {question}\\nA: {answer}")`` writes the filled template into ``into``."""
    def step(row):
        return {**row, into: template.format(**row)}
    return step


def where(**equals: Any) -> Callable[[Mapping[str, Any]], bool]:
    """A predicate for ``Dataset.filter``: every named field equals its value (or is one of a set / list / tuple of values)."""
    def keep(row):
        return all(row.get(k) in v if isinstance(v, (set, list, tuple, frozenset)) else row.get(k) == v for k, v in equals.items())
    return keep


# ------------------------------------------------------------------------------------------------ token records
POLICIES = ("truncate", "truncate_left", "drop", "split", "raise")


def over_length(length: int, policy: str = "truncate", field: str = "tokens", keep_fields: bool = True) -> Callable[[Mapping[str, Any]], Iterator[Dict[str, Any]]]:
    """A ``flat_map`` step: what becomes of a record whose ``field`` holds more than ``length`` tokens.  ``truncate`` keeps the first
    ``length`` (``truncate_left`` the last - a chat's latest turns), ``drop`` yields nothing, ``split`` yields consecutive pieces of at
    most ``length``, ``raise`` refuses naming the record's length.  Per-token companions of the same length (a mask) are cut alike."""
    if policy not in POLICIES:
        raise ValueError(f"over-length policy {policy!r}; known: {POLICIES}")

    def cut(row, lo, hi, n):
        out = dict(row) if keep_fields else {}
        for k, v in row.items():
            if hasattr(v, "__len__") and not isinstance(v, (str, bytes, Mapping)) and len(v) == n:
                out[k] = v[lo:hi]
        return out

    def step(row):
        n = len(row[field])
        if n <= length:
            yield row
        elif policy == "truncate":
            yield cut(row, 0, length, n)
        elif policy == "truncate_left":
            yield cut(row, n - length, n, n)
        elif policy == "split":
            for lo in range(0, n, length):
                yield cut(row, lo, min(n, lo + length), n)
        elif policy == "raise":
            raise ValueError(f"a record holds {n} tokens in {field!r}, the chain reads at most {length}")
    return step


def require_length(length: int, field: str = "tokens") -> Callable[[Mapping[str, Any]], Mapping[str, Any]]:
    def step(row):
        if len(row[field]) != length:
            raise ValueError(f"a record holds {len(row[field])} tokens in {field!r}, the chain was promised {length}")
        return row
    return step


def target_count(row: Mapping[str, Any], field: str = "tokens", mask: str = "mask") -> int:
    """How many targets a causal row trains on: its masked places past the first token, or all but the first."""
    if mask in row:
        return int(np.asarray(row[mask])[1:].sum())
    return max(0, len(row[field]) - 1)


def causal_windows(window: int, field: str = "tokens", stride: Optional[int] = None, min_targets: int = 1) -> Callable[[Mapping[str, Any]], Iterator[Dict[str, Any]]]:
    """A ``flat_map`` step: a document of ``n`` tokens becomes rows of at most ``window + 1`` tokens (``window`` inputs and their
    targets), each starting on the last token of the one before, so the boundary token is an input once and a target once.  ``stride``
    below ``window`` overlaps the windows further (context for the first targets of a window); the overlapped targets are then masked out
    (``mask``), so every target is still trained on once."""
    stride = stride or window
    if not 0 < stride <= window:
        raise ValueError(f"stride {stride} outside (0, window = {window}]")

    def step(row):
        toks = np.asarray(row[field])
        n = len(toks)
        start, covered = 0, 0                                   # covered: targets up to this index are already trained on
        while start < n - 1:
            piece = toks[start:start + window + 1]
            mask = np.zeros(len(piece), dtype=np.int64)
            first_new = max(1, covered + 1 - start)
            mask[first_new:] = 1
            if mask.sum() >= min_targets:
                yield {**row, field: piece, "mask": mask, "offset": start}
            covered = start + len(piece) - 1
            if start + window + 1 >= n:
                break
            start += stride
    return step
