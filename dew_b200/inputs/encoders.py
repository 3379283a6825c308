"""Encoders that turn raw conditioning data into the value a model keyword takes.

An encoder tokenises on the host (in the data workers, or before a sampling call) and encodes on the device.  ``ConditionEncoder``
is the contract: ``tokenize(texts) -> {"tokens", "mask"}``, ``encode(tokens, mask) -> context`` (a mapping with ``text [B, T, d]``,
``mask [B, T]`` and, where the tower pools, ``pooled [B, d]``), ``null(rows)`` the tokens that stand for "no condition", and
``record()`` / ``ConditionEncoder.bound(record)`` so a run can write down which encoder it used and rebuild it.

``CharTable`` encodes text as a table lookup - one id per character, one fixed random vector per id: it costs nothing and needs no
files, so tests, benchmarks and smoke runs use it as their text encoder; its output has the form of a real tower's.
``TowerEncoder`` wraps a text tower of ``dew_b200.models.encoders`` (CLIP / SigLIP / T5) with its tokenizer.
``encode_conditions`` runs a spec's encoders over a batch: the one encoding a training step and a sampling task share.

Reference: src/dew/inputs/condition.py (``ConditionEncoder``), src/dew/inputs/encoders.py (``char_codes``, ``CharTable``),
src/dew/inputs/spec.py (``encode_conditions``, ``TextCondition``).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence

import torch
import torch.nn as nn

_ENCODERS: Dict[str, type] = {}


def encoder(name: str):
    def wrap(cls):
        _ENCODERS[name] = cls
        cls.record_name = name
        return cls
    return wrap


class ConditionEncoder(nn.Module):
    record_name = ""

    def tokenize(self, texts: Sequence[str]) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def encode(self, tokens: torch.Tensor, mask: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def null(self, rows: int) -> Dict[str, torch.Tensor]:
        return self.tokenize([""] * rows)

    def forward(self, tokens, mask=None):
        return self.encode(tokens, mask)

    def recorded_fields(self) -> Dict[str, Any]:
        return {}

    def record(self) -> Dict[str, Any]:
        return {"class": self.record_name, "fields": self.recorded_fields()}

    @staticmethod
    def bound(record: Mapping[str, Any]) -> "ConditionEncoder":
        name = record.get("class")
        if name not in _ENCODERS:
            raise KeyError(f"unknown condition encoder {name!r}; known: {sorted(_ENCODERS)}")
        return _ENCODERS[name](**record.get("fields", {}))


def char_codes(texts: Sequence[str], tokens: int, vocab: int) -> Dict[str, torch.Tensor]:
    """Each text as ``tokens`` ids of a ``vocab``-row table behind a start token (id 1; 0 pads), with its mask."""
    ids = torch.zeros(len(texts), tokens, dtype=torch.long)
    mask = torch.zeros(len(texts), tokens, dtype=torch.bool)
    for i, t in enumerate(texts):
        row = [1] + [2 + (ord(c) % (vocab - 2)) for c in t][: tokens - 1]
        ids[i, : len(row)] = torch.tensor(row)
        mask[i, : len(row)] = True
    return {"tokens": ids, "mask": mask}


@encoder("char_table")
class CharTable(ConditionEncoder):
    def __init__(self, features: int = 64, tokens: int = 32, vocab: int = 258, seed: int = 0, pooled: bool = True):
        super().__init__()
        self.features, self.tokens, self.vocab, self.seed, self.pooled = features, tokens, vocab, seed, pooled
        g = torch.Generator().manual_seed(seed)
        self.register_buffer("table", torch.randn(vocab, features, generator=g) * (features ** -0.5) * 4.0)

    def tokenize(self, texts):
        return char_codes(texts, self.tokens, self.vocab)

    def encode(self, tokens, mask=None):
        text = self.table[tokens]
        mask = (tokens != 0) if mask is None else mask.bool()
        text = text * mask[..., None]
        out = {"text": text, "mask": mask}
        if self.pooled:
            out["pooled"] = text.sum(1) / mask.sum(1, keepdim=True).clamp_min(1)
        return out

    def recorded_fields(self):
        return {"features": self.features, "tokens": self.tokens, "vocab": self.vocab, "seed": self.seed, "pooled": self.pooled}


class TowerEncoder(ConditionEncoder):
    """A frozen text tower with its tokenizer: ``tower(ids, key_mask) -> (tokens' states, pooled)`` as ``models.encoders.TextTower``
    and ``T5Encoder`` return them."""
    record_name = "tower"

    def __init__(self, tower: nn.Module, tokenizer: Callable[[Sequence[str]], Dict[str, torch.Tensor]], trainable: bool = False):
        super().__init__()
        self.tower, self._tokenize = tower, tokenizer
        if not trainable:
            for p in tower.parameters():
                p.requires_grad_(False)
        self.trainable = trainable

    def tokenize(self, texts):
        return self._tokenize(list(texts))

    def encode(self, tokens, mask=None):
        ctx = torch.enable_grad() if self.trainable else torch.no_grad()
        with ctx:
            out = self.tower(tokens, mask)
        states, pooled = out if isinstance(out, tuple) else (out, None)
        res = {"text": states, "mask": (tokens != 0) if mask is None else mask.bool()}
        if pooled is not None:
            res["pooled"] = pooled
        return res


def encode_conditions(conditions: Mapping[str, Any], batch: Mapping[str, Any], device=None) -> Dict[str, Any]:
    """Each condition of a spec (``InputSpec.conditions``: keyword -> ``Condition``) encoded from the batch: a condition whose
    encoder is a ``ConditionEncoder`` reads ``<field>`` (ids) and ``<field>_mask``; raw captions under ``<field>_text`` are tokenised
    first; any other callable encoder is applied to the field as it is."""
    out: Dict[str, Any] = {}
    for keyword, cond in conditions.items():
        key = cond.field.key
        enc = cond.encoder
        if isinstance(enc, ConditionEncoder):
            if key not in batch and f"{key}_text" in batch:
                tok = enc.tokenize(batch[f"{key}_text"])
                tokens, mask = tok["tokens"], tok.get("mask")
            else:
                tokens, mask = batch[key], batch.get(f"{key}_mask")
            if device is not None:
                tokens, mask = tokens.to(device), None if mask is None else mask.to(device)
            out[keyword] = enc.encode(tokens, mask)
        elif key in batch:
            v = batch[key]
            out[keyword] = enc(v) if enc is not None else v
    return out
