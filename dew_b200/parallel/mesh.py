"""Mesh axes and ``MeshSpec``: how the GPUs of a job are factored into parallelism axes.

Seven named axes as in the reference (src/dew/mesh.py:18-39; ``MeshSpec`` src/dew/distributed/placement.py:142-254):
``('diloco', 'data', 'expert', 'fsdp', 'tensor', 'sequence', 'stage')``; ``data`` takes whatever the others leave.
Here each axis becomes a ``torch.distributed`` process group over one process per GPU; on one NVSwitch box every
axis has the same link bandwidth, so the axis order only fixes which ranks are neighbours.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

AXES = ("diloco", "data", "expert", "fsdp", "tensor", "sequence", "stage")
BATCH_AXES = ("data", "expert", "fsdp")


class LayoutRefused(ValueError):
    """A layout cannot be placed on the mesh; the message lists every reason."""


@dataclass(frozen=True)
class MeshSpec:
    fsdp: int = 1
    expert: int = 1
    tensor: int = 1
    sequence: int = 1
    stage: int = 1
    replicas: int = 1          # HSDP: replicas of the fsdp group
    diloco: int = 1
    explicit: Tuple[Tuple[str, int], ...] = ()
    devices: Optional[int] = None

    def sizes(self, world: Optional[int] = None) -> Dict[str, int]:
        world = world if world is not None else (self.devices or (dist.get_world_size() if dist.is_initialized() else 1))
        fixed = self.fsdp * self.expert * self.tensor * self.sequence * self.stage * self.diloco
        if world % fixed:
            raise LayoutRefused(f"{world} devices do not factor into fsdp={self.fsdp} expert={self.expert} "
                                f"tensor={self.tensor} sequence={self.sequence} stage={self.stage} diloco={self.diloco}")
        data = world // fixed
        if self.replicas > 1:
            if data % self.replicas and data != 1:
                raise LayoutRefused(f"replicas={self.replicas} does not divide the {data}-way data axis")
            data = max(data, self.replicas)
        sizes = {"diloco": self.diloco, "data": data, "expert": self.expert, "fsdp": self.fsdp, "tensor": self.tensor,
                 "sequence": self.sequence, "stage": self.stage}
        for name, n in self.explicit:
            sizes[name] = n
        return sizes

    def world(self) -> int:
        s = self.sizes()
        n = 1
        for v in s.values():
            n *= v
        return n

    def data_size(self) -> int:
        return self.sizes()["data"]

    def build(self, devices: Optional[int] = None) -> "Mesh":
        return Mesh(self, devices)


class Mesh:
    """Rank coordinates and per-axis process groups.  Groups are created lazily and only when torch.distributed is
    initialised; on one process every axis has size 1 and no group is made."""

    def __init__(self, spec: MeshSpec, devices: Optional[int] = None):
        self.spec = spec
        self.world = devices or (dist.get_world_size() if dist.is_initialized() else (spec.devices or 1))
        self.sizes = spec.sizes(self.world)
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.shape = tuple(self.sizes[a] for a in AXES)
        self._groups: Dict[Tuple[str, ...], Optional[dist.ProcessGroup]] = {}

    def coords(self, rank: Optional[int] = None) -> Dict[str, int]:
        r = self.rank if rank is None else rank
        out = {}
        for a in reversed(AXES):
            out[a] = r % self.sizes[a]
            r //= self.sizes[a]
        return out

    def rank_of(self, coords: Dict[str, int]) -> int:
        r = 0
        for a in AXES:
            r = r * self.sizes[a] + coords[a]
        return r

    def axis_ranks(self, axes: Sequence[str], rank: Optional[int] = None) -> List[int]:
        """Ranks that differ from ``rank`` only along ``axes`` (ordered)."""
        base = self.coords(rank)
        ranks = [dict(base)]
        for a in axes:
            ranks = [dict(c, **{a: i}) for c in ranks for i in range(self.sizes[a])]
        return sorted(self.rank_of(c) for c in ranks)

    def size(self, *axes: str) -> int:
        n = 1
        for a in axes:
            n *= self.sizes[a]
        return n

    def group(self, *axes: str) -> Optional[dist.ProcessGroup]:
        """The process group spanning ``axes`` through this rank (None on one process or a size-1 span)."""
        key = tuple(axes)
        if key in self._groups:
            return self._groups[key]
        if not dist.is_initialized() or self.size(*axes) == 1:
            self._groups[key] = None
            return None
        mine = None
        seen = set()
        for r in range(self.world):           # every rank creates every group in the same order
            members = tuple(self.axis_ranks(axes, r))
            if members in seen:
                continue
            seen.add(members)
            g = dist.new_group(list(members))
            if self.rank in members:
                mine = g
        self._groups[key] = mine
        return mine

    def index(self, *axes: str) -> int:
        """This rank's linear index within the span of ``axes``."""
        return self.axis_ranks(axes).index(self.rank)
