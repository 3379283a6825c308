"""Typed kernel selection with reasons.

Each op owns an ordered list of kernels; each kernel an ordered list of requirements.  The first kernel whose
requirements all hold takes the call.  Forcing a kernel that refuses raises :class:`KernelRefused` listing every
refusal, and :func:`explain` returns the same report without raising (the idea of
src/dew/nn/kernels/selection.py:1-60,113-300, restated for one backend: the sm_100a kernel or the library arm).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple


class KernelRefused(RuntimeError):
    pass


@dataclass(frozen=True)
class Requirement:
    code: str
    predicate: Callable[[Dict[str, Any]], bool]
    detail: str = ""


@dataclass
class Kernel:
    name: str
    requirements: Sequence[Requirement] = ()
    receipt: str = ""      # measured evidence for this kernel's place in the order

    def refusals(self, case: Dict[str, Any]) -> List[str]:
        out = []
        for r in self.requirements:
            try:
                ok = bool(r.predicate(case))
            except Exception as e:  # a predicate that cannot evaluate refuses
                ok = False
                out.append(f"{r.code}: predicate failed ({e})")
                continue
            if not ok:
                out.append(f"{r.code}: {r.detail}")
        return out


@dataclass
class Op:
    name: str
    kernels: List[Kernel] = field(default_factory=list)
    declared: Dict[Tuple, str] = field(default_factory=dict)   # cell key -> kernel name chosen by measurement

    def select(self, case: Dict[str, Any], forced: Optional[str] = None, cell: Optional[Tuple] = None) -> str:
        forced = forced or os.environ.get(f"DEWB_KERNEL_{self.name.upper()}")
        reasons: Dict[str, List[str]] = {}
        order = list(self.kernels)
        if cell is not None and cell in self.declared:
            order.sort(key=lambda k: 0 if k.name == self.declared[cell] else 1)
        for k in order:
            if forced and k.name != forced:
                continue
            why = k.refusals(case)
            if not why:
                return k.name
            reasons[k.name] = why
        if forced and forced not in [k.name for k in self.kernels]:
            raise KernelRefused(f"{self.name}: unknown kernel {forced!r}; known {[k.name for k in self.kernels]}")
        raise KernelRefused(f"{self.name}: no kernel takes {case}: {reasons}")

    def explain(self, case: Dict[str, Any]) -> Dict[str, List[str]]:
        return {k.name: k.refusals(case) for k in self.kernels}


OPS: Dict[str, Op] = {}


def op(name: str) -> Op:
    return OPS.setdefault(name, Op(name))
