"""Counter-based keys: every random draw is named by (run key, step, example index, purpose).

The reference derives a per-example key by folding the run key with the step and the example's
global index so that a batch's draws do not depend on sharding or microbatching
(src/dew/objectives/base.py:411-581).  Here a key is a 64-bit integer; folding is a SplitMix64
style mix, and draws are produced row by row from per-row generators, so a row's noise is the same
whichever rank or microbatch holds it.
"""
from __future__ import annotations

import hashlib
from typing import Iterable, Sequence, Union

import torch

MASK = (1 << 64) - 1
Key = int


def _mix(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK
    return x ^ (x >> 31)


def key(seed: Union[int, str]) -> Key:
    if isinstance(seed, str):
        seed = int.from_bytes(hashlib.sha256(seed.encode()).digest()[:8], "little")
    return _mix(int(seed) & MASK)


def fold_in(k: Key, data: Union[int, str]) -> Key:
    if isinstance(data, str):
        data = int.from_bytes(hashlib.sha256(data.encode()).digest()[:8], "little")
    return _mix((k ^ _mix(int(data) & MASK)) & MASK)


def split(k: Key, n: int = 2) -> Sequence[Key]:
    return [fold_in(k, i + 1) for i in range(n)]


def generator(k: Key, device: Union[str, torch.device] = "cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(k & ((1 << 63) - 1))
    return g


def normal(k: Key, shape: Iterable[int], dtype=torch.float32, device="cpu") -> torch.Tensor:
    return torch.randn(tuple(shape), generator=generator(k, device), dtype=dtype, device=device)


def uniform(k: Key, shape: Iterable[int], low=0.0, high=1.0, dtype=torch.float32, device="cpu") -> torch.Tensor:
    u = torch.rand(tuple(shape), generator=generator(k, device), dtype=dtype, device=device)
    return u * (high - low) + low


def randint(k: Key, shape: Iterable[int], low: int, high: int, device="cpu") -> torch.Tensor:
    return torch.randint(low, high, tuple(shape), generator=generator(k, device), device=device)


def per_example(k: Key, indices: Sequence[int], draw, shape: Iterable[int], **kw) -> torch.Tensor:
    """Stack one independent draw per example, each keyed by the example's global index."""
    rows = [draw(fold_in(k, int(i)), shape, **kw) for i in indices]
    return torch.stack(rows, 0)
