"""What a corpus holds, measured before a run spends compute on it: token-length statistics, how well it packs, how much of the
vocabulary it uses, exact and near duplicates, and how much a context length cuts.

``length_report(lengths, seq_len)``   count, mean, percentiles, the share of documents and of tokens a window of ``seq_len`` cuts
``packing_report(lengths, seq_len)``  the real-token share of first-fit-decreasing packed windows against padding each to ``seq_len``
``vocabulary_report(docs, vocab)``    the tokens used, the coverage of the vocabulary, the most frequent tokens' share
``duplicates(texts)``                 exact duplicates by hash and near duplicates by MinHash over character shingles
``analyse(dataset, tokenizer, ...)``  all of the above over a sample of a dataset, as one JSON-able report

Reference: src/dew/data/analysis.py (corpus facts reported before training), src/dew/data/facts.py.
"""
from __future__ import annotations

import hashlib
from typing import Any, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import numpy as np


def length_report(lengths: Sequence[int], seq_len: Optional[int] = None) -> Dict[str, float]:
    a = np.asarray(list(lengths), dtype=np.int64)
    if a.size == 0:
        return {"documents": 0}
    out = {"documents": int(a.size), "tokens": int(a.sum()), "mean": float(a.mean()), "min": int(a.min()), "max": int(a.max()),
           **{f"p{p}": float(np.percentile(a, p)) for p in (50, 90, 99)}}
    if seq_len:
        over = a > seq_len
        out["cut_documents"] = float(over.mean())
        out["cut_tokens"] = float((a[over] - seq_len).sum() / max(1, a.sum()))
    return out


def packing_report(lengths: Sequence[int], seq_len: int) -> Dict[str, float]:
    a = np.minimum(np.asarray(list(lengths), dtype=np.int64), seq_len)
    order = np.sort(a)[::-1]
    room: List[int] = []
    for n in order.tolist():
        for i in range(len(room)):
            if room[i] >= n:
                room[i] -= n
                break
        else:
            room.append(seq_len - n)
    windows = max(1, len(room))
    return {"windows": len(room), "real_token_share": float(a.sum() / (windows * seq_len)),
            "padded_real_token_share": float(a.sum() / max(1, a.size * seq_len)), "windows_saved": float(1 - windows / max(1, a.size))}


def vocabulary_report(docs: Iterable[Sequence[int]], vocab_size: int, top: int = 10) -> Dict[str, Any]:
    counts = np.zeros(vocab_size, dtype=np.int64)
    for d in docs:
        ids = np.asarray(d, dtype=np.int64)
        if ids.size:
            if ids.min() < 0 or ids.max() >= vocab_size:
                raise ValueError(f"a token id outside the vocabulary of {vocab_size}")
            counts += np.bincount(ids, minlength=vocab_size)
    total = int(counts.sum())
    order = np.argsort(-counts)[:top]
    p = counts[counts > 0] / max(1, total)
    return {"tokens": total, "used": int((counts > 0).sum()), "coverage": float((counts > 0).mean()),
            "entropy_bits": float(-(p * np.log2(p)).sum()) if total else 0.0,
            "top": [(int(i), float(counts[i] / max(1, total))) for i in order if counts[i] > 0]}


def _shingles(text: str, k: int = 5) -> set:
    t = " ".join(text.lower().split())
    return {t[i:i + k] for i in range(max(1, len(t) - k + 1))}


def minhash(text: str, hashes: int = 64, k: int = 5) -> np.ndarray:
    sig = np.full(hashes, np.iinfo(np.uint64).max, dtype=np.uint64)
    for s in _shingles(text, k):
        h = int.from_bytes(hashlib.blake2b(s.encode(), digest_size=8).digest(), "little")
        # a family of hashes from one: h_i = (a_i h + b_i) mod 2^64 with fixed odd a_i
        vals = (np.arange(1, hashes + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15) | np.uint64(1)) * np.uint64(h) \
            + np.arange(hashes, dtype=np.uint64) * np.uint64(0xC2B2AE3D27D4EB4F)
        sig = np.minimum(sig, vals)
    return sig


def duplicates(texts: Sequence[str], threshold: float = 0.8, hashes: int = 64, bands: int = 16) -> Dict[str, Any]:
    """Exact duplicates (same normalised text) and near duplicates: pairs whose MinHash signatures agree on at least
    ``threshold`` of their hashes, found through banded buckets (LSH) rather than all pairs."""
    exact: Dict[str, List[int]] = {}
    for i, t in enumerate(texts):
        exact.setdefault(hashlib.blake2b(" ".join(t.split()).encode(), digest_size=16).hexdigest(), []).append(i)
    exact_groups = [g for g in exact.values() if len(g) > 1]
    firsts = sorted(g[0] for g in exact.values())
    sigs = {i: minhash(texts[i], hashes) for i in firsts}
    rows = hashes // bands
    buckets: Dict[Tuple[int, bytes], List[int]] = {}
    for i, s in sigs.items():
        for b in range(bands):
            buckets.setdefault((b, s[b * rows:(b + 1) * rows].tobytes()), []).append(i)
    near = set()
    for members in buckets.values():
        for x in range(len(members)):
            for y in range(x + 1, len(members)):
                i, j = members[x], members[y]
                if (i, j) not in near and float((sigs[i] == sigs[j]).mean()) >= threshold:
                    near.add((i, j))
    dup_docs = sum(len(g) - 1 for g in exact_groups)
    return {"exact_groups": exact_groups, "exact_duplicate_share": dup_docs / max(1, len(texts)), "near_pairs": sorted(near)}


def analyse(dataset, tokenizer=None, *, seq_len: Optional[int] = None, text_key: str = "text", sample: int = 10000, vocab_size: Optional[int] = None
            ) -> Dict[str, Any]:
    texts, docs = [], []
    for i, row in enumerate(dataset):
        if i >= sample:
            break
        t = row[text_key] if isinstance(row, Mapping) else row
        if isinstance(t, str):
            texts.append(t)
            if tokenizer is not None:
                docs.append(list(tokenizer.encode(t)))
        else:
            docs.append(list(np.asarray(t).reshape(-1)))
    lengths = [len(d) for d in docs] if docs else [len(t) for t in texts]
    report: Dict[str, Any] = {"sampled": len(lengths), "lengths": length_report(lengths, seq_len)}
    if seq_len:
        report["packing"] = packing_report(lengths, seq_len)
    if docs and (vocab_size or getattr(tokenizer, "vocab_size", None)):
        report["vocabulary"] = vocabulary_report(docs, int(vocab_size or tokenizer.vocab_size))
    if texts:
        d = duplicates(texts)
        report["duplicates"] = {"exact_duplicate_share": d["exact_duplicate_share"], "near_pairs": len(d["near_pairs"])}
    return report
