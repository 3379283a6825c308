"""The batch a decision model reads (``DecisionInputs``) and how laid-out rows are packed into it.

Rows are packed first-fit into windows of one length: a window holds whole rows, told apart by ``segment_ids`` (0 for padding,
1.. for the rows of the window, each with positions restarting at 0), so one forward pass reads many short rows without
padding each to the longest.  Question slots are per window: a window's ``Q`` slots list the questions of its rows in window
order, each with ``K`` option slots.

Reference: src/dew/decision/inputs.py (``DecisionInputs``), src/dew/decision/task.py (``PassPlan`` first-fit placement,
``laid_out``).
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .layout import Encoded


@dataclass
class DecisionInputs:
    tokens: torch.Tensor         # [B, L] int64
    segment_ids: torch.Tensor    # [B, L] int32, 0 = padding
    positions: torch.Tensor      # [B, L] int64, restarting per row
    token_kind: torch.Tensor     # [B, L] int64, -1 = no question type at this token
    kinds: torch.Tensor          # [B, Q] int64, -1 = empty slot
    segment_of: torch.Tensor     # [B, Q] int32: the row (segment id) each question belongs to
    options: torch.Tensor        # [B, Q, K] bool: real options
    markers: torch.Tensor        # [B, Q, K] int64
    span_start: torch.Tensor     # [B, Q, K] int64
    span_end: torch.Tensor       # [B, Q, K] int64 (exclusive)
    asked_start: torch.Tensor    # [B, Q]
    asked_end: torch.Tensor      # [B, Q]
    readout: torch.Tensor        # [B, Q]
    row_end: torch.Tensor        # [B, Q] the last token of the question's row
    label_ids: Optional[torch.Tensor] = None   # [B, Q, K] int64 (lettered layouts)

    def to(self, device) -> "DecisionInputs":
        return DecisionInputs(**{f.name: (None if getattr(self, f.name) is None else getattr(self, f.name).to(device)) for f in fields(self)})

    def as_batch(self, prefix: str = "") -> Dict[str, torch.Tensor]:
        """The tensors under their field names (what a trainer splits into microbatches along dim 0)."""
        return {prefix + f.name: getattr(self, f.name) for f in fields(self) if getattr(self, f.name) is not None}

    @classmethod
    def from_batch(cls, batch, prefix: str = "") -> "DecisionInputs":
        return cls(**{f.name: batch.get(prefix + f.name) for f in fields(cls)})

    @property
    def ordinal(self) -> torch.Tensor:
        """[B, Q]: whether the question's options are ordered levels (a score)."""
        return self.kinds == 1


def first_fit(rows: Sequence[Encoded], length: int, max_windows: Optional[int] = None, questions: Optional[int] = None):
    """Place rows first-fit into windows of ``length`` tokens (and at most ``questions`` question slots each).  Returns
    ``(windows, leftover)``: per window the indices of its rows, and the indices that found no room (with ``max_windows``)."""
    room: List[int] = []
    slots: List[int] = []
    windows: List[List[int]] = []
    leftover: List[int] = []
    for i, r in enumerate(rows):
        n, q = len(r), len(r.names)
        if n > length or (questions is not None and q > questions):
            raise ValueError(f"a row of {n} tokens and {q} questions does not fit a window of {length} tokens / {questions} questions")
        for w in range(len(windows)):
            if room[w] >= n and (questions is None or slots[w] >= q):
                windows[w].append(i)
                room[w] -= n
                if questions is not None:
                    slots[w] -= q
                break
        else:
            if max_windows is not None and len(windows) >= max_windows:
                leftover.append(i)
                continue
            windows.append([i])
            room.append(length - n)
            slots.append((questions or 0) - q)
    return windows, leftover


def collate(rows: Sequence[Encoded], windows: Sequence[Sequence[int]], length: int, questions: int, options: int, pad: int = 0,
            batch: Optional[int] = None) -> Tuple[DecisionInputs, List[List[Tuple[int, int]]]]:
    """Build the tensors of ``windows`` (lists of row indices).  Also returns, per row index, where its questions went:
    ``where[i] = [(window, slot), ...]`` in the row's question order."""
    B = batch if batch is not None else len(windows)
    if len(windows) > B:
        raise ValueError(f"{len(windows)} windows do not fit a batch of {B}")
    labelled = any(r.label_ids is not None for r in rows)
    z = lambda *s, fill=0, dt=torch.int64: torch.full(s, fill, dtype=dt)
    t = dict(tokens=z(B, length, fill=pad), segment_ids=z(B, length, dt=torch.int32), positions=z(B, length), token_kind=z(B, length, fill=-1),
             kinds=z(B, questions, fill=-1), segment_of=z(B, questions, dt=torch.int32), options=torch.zeros(B, questions, options, dtype=torch.bool),
             markers=z(B, questions, options), span_start=z(B, questions, options), span_end=z(B, questions, options),
             asked_start=z(B, questions), asked_end=z(B, questions), readout=z(B, questions), row_end=z(B, questions),
             label_ids=z(B, questions, options) if labelled else None)
    where: List[List[Tuple[int, int]]] = [[] for _ in rows]
    for w, members in enumerate(windows):
        at, slot = 0, 0
        for seg, i in enumerate(members, start=1):
            r = rows[i]
            n = len(r)
            t["tokens"][w, at:at + n] = torch.tensor(r.tokens)
            t["segment_ids"][w, at:at + n] = seg
            t["positions"][w, at:at + n] = torch.arange(n)
            t["token_kind"][w, at:at + n] = torch.tensor(r.token_kind)
            for q in range(len(r.names)):
                k = r.counts[q]
                if k > options:
                    raise ValueError(f"a question of {k} options does not fit {options} option slots")
                if slot >= questions:
                    raise ValueError(f"a window's rows ask more than its {questions} question slots")
                t["kinds"][w, slot] = r.kinds[q]
                t["segment_of"][w, slot] = seg
                t["options"][w, slot, :k] = True
                t["markers"][w, slot, :k] = torch.tensor(r.markers[q]) + at
                t["span_start"][w, slot, :k] = torch.tensor([a for a, _ in r.spans[q]]) + at
                t["span_end"][w, slot, :k] = torch.tensor([b for _, b in r.spans[q]]) + at
                t["asked_start"][w, slot] = r.asked[q][0] + at
                t["asked_end"][w, slot] = r.asked[q][1] + at
                t["readout"][w, slot] = r.readout[q] + at
                t["row_end"][w, slot] = at + n - 1
                if labelled and r.label_ids is not None:
                    t["label_ids"][w, slot, :k] = torch.tensor(r.label_ids[q])
                where[i].append((w, slot))
                slot += 1
            at += n
    return DecisionInputs(**t), where
