"""Engram: hashed n-gram lookups gated into the residual stream.  A position and the few token ids before it make one n-gram of every
size from 2 to ``max_ngram``; each is hashed (multiply the look-back ids by per-layer odd multipliers, XOR them together, reduce modulo a
prime per (size, head)) into a bucket of an embedding table, so the layer owns a very large, very cheap static memory of local token
patterns that costs no attention or MLP FLOPs.  The looked-up rows are projected to a key and a value; the value enters the stream
through a gate that is the sigmoid of the sign-preserving square root of the normalised dot product between the stream and the key - a
pattern the context does not agree with stays out.  A short causal convolution over the gated values (optional) spreads a hit over the
next few positions.

Look-back stops at the start of the sequence, at a document boundary (``segment_ids``) and at a stop token; slots it does not reach hold
the pad id.  Hashing is exact integer arithmetic in int64 (ids below 2**24 and multipliers below 2**31 keep every product under 2**55),
and identical on CPU and GPU.

Reference: src/dew/nn/engram.py (``Engram``, ``PLELayer``, ``compressed_token_map``).
"""
from __future__ import annotations

import math
import unicodedata
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import Embedding, Linear, RMSNorm

_MASK64 = (1 << 64) - 1


def splitmix64(seed: int, count: int) -> List[int]:
    """``count`` values of the SplitMix64 stream from ``seed``."""
    out, x = [], seed & _MASK64
    for _ in range(count):
        x = (x + 0x9E3779B97F4A7C15) & _MASK64
        z = x
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        out.append(z ^ (z >> 31))
    return out


def odd_multipliers(seed: int, layer: int, count: int) -> List[int]:
    """Per layer, ``count`` odd multipliers below 2**31."""
    return [int(v >> 33) | 1 for v in splitmix64(seed * 0x100000001B3 + layer, count)]


def primes_below(limit: int, count: int) -> List[int]:
    """The ``count`` largest primes not above ``limit`` (distinct moduli for the (size, head) hashes)."""
    found, n = [], limit
    while len(found) < count and n >= 2:
        if all(n % p for p in range(2, int(math.isqrt(n)) + 1)):
            found.append(n)
        n -= 1
    if len(found) < count:
        raise ValueError(f"fewer than {count} primes up to {limit}")
    return found


def compressed_token_map(vocabulary: Sequence[str]) -> torch.Tensor:
    """Token id -> the id of its normalised text: case, Unicode compatibility forms and the leading-space marker folded, so surface
    variants of one word share their n-grams.  The compressed ids are dense, in order of first appearance."""
    seen, ids = {}, []
    for text in vocabulary:
        key = unicodedata.normalize("NFKC", text).replace("▁", " ").replace("Ġ", " ").strip().lower() or text
        ids.append(seen.setdefault(key, len(seen)))
    return torch.tensor(ids, dtype=torch.long)


def lookback(tokens: torch.Tensor, steps: int, pad_id: int, segment_ids: Optional[torch.Tensor] = None, stop_id: Optional[int] = None) -> torch.Tensor:
    """``[B, S, steps]``: the token at each position and the ``steps - 1`` before it, nearest first; the slots before the sequence start,
    across a document boundary, or behind a stop token hold ``pad_id``."""
    B, S = tokens.shape
    cols, alive = [tokens], torch.ones(B, S, dtype=torch.bool, device=tokens.device)
    for k in range(1, steps):
        prev = F.pad(tokens, (k, 0), value=pad_id)[:, :S]
        ok = torch.arange(S, device=tokens.device)[None, :] >= k
        if segment_ids is not None:
            ok = ok & (F.pad(segment_ids, (k, 0), value=-1)[:, :S] == segment_ids)
        if stop_id is not None:
            ok = ok & (prev != stop_id)
        alive = alive & ok                                   # once look-back stops it stays stopped
        cols.append(torch.where(alive, prev, torch.full_like(prev, pad_id)))
    return torch.stack(cols, -1)


def ngram_buckets(window: torch.Tensor, multipliers: Sequence[int], primes: torch.Tensor) -> torch.Tensor:
    """``window [B, S, n_max]`` (nearest first) -> bucket ids ``[B, S, n_max - 1, heads]``: size ``n`` hashes the first ``n`` slots,
    ``primes [n_max - 1, heads]``; the result of (size, head) lies in ``[0, primes[size, head])``."""
    mult = torch.tensor(list(multipliers), dtype=torch.long, device=window.device)
    scaled = window.long() * mult
    running, hashes = scaled[..., 0], []
    for k in range(1, window.shape[-1]):
        running = running ^ scaled[..., k]
        hashes.append(running)
    h = torch.stack(hashes, -1)                               # [B, S, n_max - 1]
    return h[..., None] % primes.to(window.device)


def signed_sqrt(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.sqrt(x.abs())


class Engram(nn.Module):
    """``h -> h + gate * value`` with the value looked up by the hashed n-grams ending at each position.

    ``buckets`` rows per (size, head) table (each reduced modulo its own prime just below it), ``heads`` hashes per n-gram size,
    ``width`` numbers per looked-up row; ``conv`` > 0 adds a depthwise causal convolution of that length over the gated values."""

    def __init__(self, features: int, vocab_size: int, layer: int = 0, max_ngram: int = 3, heads: int = 4, buckets: int = 65536, width: int = 64,
                 conv: int = 0, seed: int = 0, pad_id: int = 0, stop_id: Optional[int] = None, token_map: Optional[torch.Tensor] = None,
                 norm_eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        if max_ngram < 2:
            raise ValueError("an n-gram has at least two tokens")
        if vocab_size >= 1 << 24:
            raise ValueError("token ids must stay below 2**24 for the hash to stay exact")
        kw = dict(dtype=dtype, device=device)
        self.features, self.max_ngram, self.heads, self.pad_id, self.stop_id = features, max_ngram, heads, pad_id, stop_id
        sizes = max_ngram - 1
        primes = torch.tensor(primes_below(buckets, sizes * heads), dtype=torch.long).view(sizes, heads)
        self.register_buffer("primes", primes, persistent=False)
        self.register_buffer("offsets", (torch.arange(sizes * heads).view(sizes, heads) * buckets), persistent=False)
        self.register_buffer("token_map", token_map if token_map is not None else None, persistent=token_map is not None)
        self.multipliers = odd_multipliers(seed, layer, max_ngram)
        self.table = Embedding(sizes * heads * buckets, width, **kw)
        self.key = Linear(sizes * heads * width, features, **kw)
        self.value = Linear(sizes * heads * width, features, zero_init=True, **kw)
        self.stream_norm, self.key_norm = RMSNorm(features, norm_eps, **kw), RMSNorm(features, norm_eps, **kw)
        self.conv = nn.Conv1d(features, features, conv, groups=features, bias=False, **kw) if conv else None
        if self.conv is not None:
            nn.init.zeros_(self.conv.weight)

    def rows(self, tokens: torch.Tensor, segment_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Table rows ``[B, S, sizes, heads]`` read for ``tokens``."""
        ids = tokens if self.token_map is None else self.token_map[tokens]
        pad = self.pad_id if self.token_map is None else int(self.token_map[self.pad_id])
        stop = None if self.stop_id is None else (self.stop_id if self.token_map is None else int(self.token_map[self.stop_id]))
        window = lookback(ids, self.max_ngram, pad, segment_ids, stop)
        return ngram_buckets(window, self.multipliers, self.primes) + self.offsets

    def forward(self, h: torch.Tensor, tokens: torch.Tensor, segment_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, S, d = h.shape
        found = self.table(self.rows(tokens, segment_ids)).reshape(B, S, -1)
        key, value = self.key(found), self.value(found)
        agreement = (self.stream_norm(h).float() * self.key_norm(key).float()).sum(-1, keepdim=True) / math.sqrt(d)
        gated = (torch.sigmoid(signed_sqrt(agreement)) * value.float()).to(h.dtype)
        if self.conv is not None:
            k = self.conv.kernel_size[0]
            gated = gated + self.conv(F.pad(gated.transpose(1, 2), (k - 1, 0))).transpose(1, 2)
        return h + gated

    def extra_repr(self) -> str:
        return f"max_ngram={self.max_ngram}, heads={self.heads}, rows={self.table.num_embeddings}"
