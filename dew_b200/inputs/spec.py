"""Declarative description of what a batch holds: ``Field``, ``Condition``, ``InputSpec``.

Capability parity with src/dew/inputs/spec.py:44-215 (``unit_range``, ``Field``, ``Condition``,
``InputSpec.check/tokenize``).  A spec is a value: it opens nothing and allocates nothing.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Optional, Sequence, Tuple

import torch


def unit_range(pixels: torch.Tensor) -> torch.Tensor:
    """uint8 pixels in [0, 255] -> float32 in [-1, 1]."""
    return pixels.to(torch.float32) / 127.5 - 1.0


@dataclass(frozen=True)
class Field:
    """One named entry of a batch with its per-example shape.

    ``variable_axes`` lists axes whose extent may differ between batches (e.g. a token axis);
    ``table`` is the size of the index table when the field holds integer ids.
    """
    key: str
    shape: Tuple[int, ...]
    variable_axes: Tuple[int, ...] = ()
    table: Optional[int] = None
    dtype: Any = None

    @classmethod
    def indexing(cls, key: str, shape: Sequence[int], model: Any) -> "Field":
        table = getattr(model, "vocab_size", None) or getattr(model, "num_classes", None)
        return cls(key, tuple(shape), table=table, dtype=torch.long)

    def check(self, value: torch.Tensor) -> None:
        got = tuple(value.shape[1:])
        if len(got) != len(self.shape):
            raise ValueError(f"field {self.key!r}: rank {len(got)} per example, declared {len(self.shape)}")
        for axis, (g, d) in enumerate(zip(got, self.shape)):
            if axis in self.variable_axes:
                continue
            if g != d:
                raise ValueError(f"field {self.key!r}: axis {axis} is {g}, declared {d}")
        if self.table is not None and value.numel() and not value.dtype.is_floating_point:
            hi = int(value.max())
            if hi >= self.table or int(value.min()) < 0:
                raise ValueError(f"field {self.key!r}: index {hi} outside table of {self.table}")


@dataclass(frozen=True)
class Condition:
    """A conditioning input: its field, an optional encoder and its drop probability for CFG."""
    field: Field
    encoder: Optional[Callable[[Any], torch.Tensor]] = None
    dropout: Optional[float] = None
    null: Optional[Any] = None          # value standing for "unconditional"
    tokenizer: Optional[Any] = None


@dataclass(frozen=True)
class InputSpec:
    sample: Field
    conditions: Mapping[str, Condition] = field(default_factory=dict)
    mask: Optional[Field] = None

    def check(self, batch: Mapping[str, torch.Tensor]) -> None:
        if self.sample.key not in batch:
            raise KeyError(f"batch has no {self.sample.key!r}; it holds {sorted(batch)}")
        self.sample.check(batch[self.sample.key])
        for name, cond in self.conditions.items():
            if cond.field.key in batch:
                cond.field.check(batch[cond.field.key])
        if self.mask is not None and self.mask.key in batch:
            self.mask.check(batch[self.mask.key])

    def tokenize(self, captions: Sequence[str]) -> Mapping[str, torch.Tensor]:
        out = {}
        for name, cond in self.conditions.items():
            if cond.tokenizer is not None:
                length = cond.field.shape[0]
                rows = [list(cond.tokenizer.encode(c))[:length] for c in captions]
                pad = getattr(cond.tokenizer, "pad_id", 0)
                out[cond.field.key] = torch.tensor([r + [pad] * (length - len(r)) for r in rows], dtype=torch.long)
        return out
