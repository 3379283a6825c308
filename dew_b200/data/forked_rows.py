"""Rows that share a prefix, computed once.  A scoring or training call often holds rows that begin alike: a prompt's sampled
completions, a preference pair's two halves, one state's questions.  Laid out whole, every row computes the prefix again.
``ForkedRows.pack`` groups rows by their longest common prefix, lays each group's prefix once as a document and each row's rest as a
document continuing it, and packs the groups first-fit into windows.  ``Forks`` carries, per token, its document and its document's
parent; attention lets a token see its own document causally and all of its parent - so every row's tokens compute exactly what they
would in the row laid out alone, the prefix's FLOPs paid once per group.  ``gathered`` maps the windows' outputs back to each row's own
layout; a gradient through that map sums a shared token's cotangent over the rows that hold it, as the rows laid out whole would.

A model reads the windows as packed rows: ``model(tokens, positions=packed.positions, segment_ids=packed.forks)``.  Softmax attention
takes ``Forks`` where it takes segment ids (the score-matrix form); a recurrent mixer does not - a state cannot fork without being copied
- and such a model lays its rows whole (``share=False``) through the same packer.

Reference: src/dew/data/forked_rows.py (``ForkedRows``), src/dew/batch.py (``Forks``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch


@dataclass
class Forks:
    """Per token: ``segment_ids`` - its document (-1: padding); ``parent_ids`` - the document its document continues (-1: none)."""
    segment_ids: torch.Tensor
    parent_ids: torch.Tensor

    def visible(self) -> torch.Tensor:
        """``[B, S, S]``: query i sees key j when j is not later and sits in i's document or in its parent."""
        seg, par = self.segment_ids, self.parent_ids
        S = seg.shape[1]
        earlier = torch.ones(S, S, dtype=torch.bool, device=seg.device).tril()
        real = (seg >= 0)
        own = seg[:, :, None] == seg[:, None, :]
        parent = (par[:, :, None] == seg[:, None, :]) & (par[:, :, None] >= 0)
        return (own | parent) & earlier & real[:, :, None] & real[:, None, :]

    def to(self, device) -> "Forks":
        return Forks(self.segment_ids.to(device), self.parent_ids.to(device))


def common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


def group_by_prefix(rows: Sequence[Sequence[int]], min_prefix: int = 1) -> List[Tuple[int, List[int]]]:
    """``(prefix length, row indices)`` per group.  Rows are visited in lexicographic order, where rows that begin alike are neighbours; a
    row joins the open group while the group's common prefix with it stays at least ``min_prefix`` long.  A prefix always leaves every row
    of its group at least one token of its own."""
    order = sorted(range(len(rows)), key=lambda i: list(rows[i]))
    groups: List[Tuple[int, List[int]]] = []
    for i in order:
        if groups:
            p, members = groups[-1]
            first = rows[members[0]]
            shared = min(common_prefix(first[:p] if len(members) > 1 else first, rows[i]), len(rows[i]) - 1, min(len(rows[m]) for m in members) - 1)
            if shared >= max(1, min_prefix):
                groups[-1] = (shared, members + [i])
                continue
        groups.append((0, [i]))
    return groups


@dataclass
class ForkedRows:
    tokens: torch.Tensor            # [W, window]
    positions: torch.Tensor         # [W, window]: a token's position in its own row
    forks: Forks
    slots: List[torch.Tensor]       # per row: flat indices into [W * window] of its tokens, in the row's order
    lengths: List[int]
    laid: int                       # tokens laid out (without padding)
    whole: int                      # tokens the rows hold laid out whole

    @staticmethod
    def pack(rows: Sequence[Sequence[int]], window: int, share: bool = True, min_prefix: int = 1, pad_id: int = 0) -> "ForkedRows":
        rows = [list(r) for r in rows]
        if any(len(r) == 0 for r in rows):
            raise ValueError("an empty row has no tokens to lay out")
        too_long = [i for i, r in enumerate(rows) if len(r) > window]
        if too_long:
            raise ValueError(f"row {too_long[0]} holds {len(rows[too_long[0]])} tokens, a window {window}")
        groups = group_by_prefix(rows, min_prefix) if share else [(0, [i]) for i in range(len(rows))]
        final: List[Tuple[int, List[int]]] = []
        for p, members in groups:                                  # a group that cannot fit one window lays its rows whole
            size = p + sum(len(rows[m]) - p for m in members)
            final += [(p, members)] if size <= window else [(0, [m]) for m in members]
        sized = sorted(((p + sum(len(rows[m]) - p for m in ms), p, ms) for p, ms in final), key=lambda g: -g[0])
        room: List[int] = []
        placed: List[List[Tuple[int, List[int]]]] = []
        for size, p, ms in sized:                                  # first fit, largest first
            for w, free in enumerate(room):
                if size <= free:
                    room[w] -= size
                    placed[w].append((p, ms))
                    break
            else:
                room.append(window - size)
                placed.append([(p, ms)])
        W = len(placed)
        tokens = torch.full((W, window), pad_id, dtype=torch.long)
        positions = torch.zeros((W, window), dtype=torch.long)
        seg = torch.full((W, window), -1, dtype=torch.long)
        par = torch.full((W, window), -1, dtype=torch.long)
        slots: List[Optional[torch.Tensor]] = [None] * len(rows)
        for w, groups_here in enumerate(placed):
            at, doc = 0, 0
            for p, ms in groups_here:
                prefix_at, prefix_doc = at, doc
                if p:
                    tokens[w, at:at + p] = torch.tensor(rows[ms[0]][:p])
                    positions[w, at:at + p] = torch.arange(p)
                    seg[w, at:at + p] = doc
                    at, doc = at + p, doc + 1
                for m in ms:
                    rest = rows[m][p:]
                    n = len(rest)
                    tokens[w, at:at + n] = torch.tensor(rest)
                    positions[w, at:at + n] = torch.arange(p, p + n)
                    seg[w, at:at + n] = doc
                    if p:
                        par[w, at:at + n] = prefix_doc
                    slots[m] = w * window + torch.cat([torch.arange(prefix_at, prefix_at + p), torch.arange(at, at + n)])
                    at, doc = at + n, doc + 1
        laid = int((seg >= 0).sum())
        return ForkedRows(tokens, positions, Forks(seg, par), slots, [len(r) for r in rows], laid, sum(len(r) for r in rows))

    def gathered(self, outputs: torch.Tensor) -> List[torch.Tensor]:
        """``outputs [W, window, ...]`` -> per row ``[len(row), ...]``, in the row's own order."""
        flat = outputs.reshape(-1, *outputs.shape[2:])
        return [flat.index_select(0, s.to(outputs.device)) for s in self.slots]

    def padded(self, outputs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``[rows, longest, ...]`` and the mask of real places."""
        parts = self.gathered(outputs)
        longest = max(self.lengths)
        out = outputs.new_zeros((len(parts), longest, *outputs.shape[2:]))
        mask = torch.zeros(len(parts), longest, dtype=torch.bool, device=outputs.device)
        for i, p in enumerate(parts):
            out[i, :p.shape[0]] = p
            mask[i, :p.shape[0]] = True
        return out, mask

    @property
    def saved(self) -> float:
        """The share of the rows' tokens the shared layout does not compute."""
        return 1.0 - self.laid / max(1, self.whole)
