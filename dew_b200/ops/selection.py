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
    routes: Dict[str, Dict[str, Any]] = field(default_factory=dict)   # kernel name -> call counts and refusal codes seen

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
                self._record(k.name, reasons, forced, cell)
                return k.name
            reasons[k.name] = why
        if forced and forced not in [k.name for k in self.kernels]:
            raise KernelRefused(f"{self.name}: unknown kernel {forced!r}; known {[k.name for k in self.kernels]}")
        raise KernelRefused(f"{self.name}: no kernel takes {case}: {reasons}")

    def explain(self, case: Dict[str, Any]) -> Dict[str, List[str]]:
        return {k.name: k.refusals(case) for k in self.kernels}

    def _record(self, chosen: str, refused: Dict[str, List[str]], forced: Optional[str], cell: Optional[Tuple]) -> None:
        """Route bookkeeping: how often each kernel took a call and, when an earlier kernel in the order refused, why."""
        row = self.routes.setdefault(chosen, {"calls": 0, "forced": 0, "declared_cell": 0, "after_refusals": {}})
        row["calls"] += 1
        row["forced"] += 1 if forced else 0
        row["declared_cell"] += 1 if (cell is not None and cell in self.declared) else 0
        for name, why in refused.items():
            for w in why:
                key = f"{name}: {w.split(':')[0]}"
                row["after_refusals"][key] = row["after_refusals"].get(key, 0) + 1


OPS: Dict[str, Op] = {}


def op(name: str) -> Op:
    return OPS.setdefault(name, Op(name))


def route_report(reset: bool = False) -> Dict[str, Dict[str, Dict[str, Any]]]:
    """Per op, which kernels took how many calls since the process started (or the last reset), how many of those were forced
    or came from a measured cell, and which refusals of earlier kernels sent calls there - the run-time view of the selector
    (the reference's route report: tools/kernel_routes.py, src/dew/nn/kernels/selection.py)."""
    out = {name: {k: dict(v, after_refusals=dict(v["after_refusals"])) for k, v in o.routes.items()} for name, o in OPS.items() if o.routes}
    if reset:
        for o in OPS.values():
            o.routes.clear()
    return out


def format_route_report(report: Optional[Dict[str, Dict[str, Dict[str, Any]]]] = None) -> str:
    report = route_report() if report is None else report
    lines = []
    for op_name in sorted(report):
        lines.append(op_name)
        for kernel, row in sorted(report[op_name].items(), key=lambda kv: -kv[1]["calls"]):
            extra = "".join(f"; {n} after {why}" for why, n in sorted(row["after_refusals"].items(), key=lambda kv: -kv[1]))
            lines.append(f"  {kernel:<16} {row['calls']:>8} calls ({row['forced']} forced, {row['declared_cell']} by measured cell){extra}")
    return "\n".join(lines)
