"""A span tracer for training and serving loops, and the reading of a trace: where a step's time went.

``Tracer.span(name)`` times a region on the host and - when CUDA is available - on the device too (a pair of CUDA events on the
current stream, resolved lazily so tracing never synchronises the loop).  ``Tracer.export(path)`` writes the spans in the Chrome /
Perfetto trace format (one host track, one device track per process); ``summary()`` totals them per name; ``breakdown(spans)``
splits the device time of a trace into compute, collective and idle time given which names are collectives.
``merge`` joins the traces of several ranks into one file, one process per rank.

An idle tracer (``enabled=False``, the default outside a capture window) costs one attribute read per span.

Reference: src/dew/telemetry/trace.py (device compute vs collectives vs idle from a capture), src/dew/telemetry/records.py.
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch


@dataclass
class Span:
    name: str
    start_us: float
    host_us: float
    device_us: Optional[float] = None
    depth: int = 0
    args: Dict[str, Any] = field(default_factory=dict)


class Tracer:
    def __init__(self, enabled: bool = False, device_time: bool = True, rank: int = 0, clock=time.perf_counter):
        self.enabled, self.rank, self.clock = enabled, rank, clock
        self.device_time = device_time and torch.cuda.is_available()
        self.spans: List[Span] = []
        self._pending: List[Tuple[Span, Any, Any]] = []
        self._depth = threading.local()
        self._t0 = clock()

    @contextlib.contextmanager
    def span(self, name: str, **args):
        if not self.enabled:
            yield None
            return
        depth = getattr(self._depth, "value", 0)
        self._depth.value = depth + 1
        ev = None
        if self.device_time:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        began = self.clock()
        s = Span(name, (began - self._t0) * 1e6, 0.0, None, depth, dict(args))
        try:
            yield s
        finally:
            s.host_us = (self.clock() - began) * 1e6
            if ev is not None:
                ev[1].record()
                self._pending.append((s, ev[0], ev[1]))
            self.spans.append(s)
            self._depth.value = depth

    def resolve(self) -> None:
        """Read the device times of finished spans (waits for their events)."""
        for s, a, b in self._pending:
            b.synchronize()
            s.device_us = a.elapsed_time(b) * 1e3
        self._pending.clear()

    def summary(self) -> Dict[str, Dict[str, float]]:
        self.resolve()
        out: Dict[str, Dict[str, float]] = {}
        for s in self.spans:
            row = out.setdefault(s.name, {"count": 0, "host_us": 0.0, "device_us": 0.0})
            row["count"] += 1
            row["host_us"] += s.host_us
            row["device_us"] += s.device_us or 0.0
        return out

    def events(self) -> List[Dict[str, Any]]:
        self.resolve()
        ev: List[Dict[str, Any]] = [{"ph": "M", "pid": self.rank, "tid": 0, "name": "thread_name", "args": {"name": "host"}},
                                    {"ph": "M", "pid": self.rank, "tid": 1, "name": "thread_name", "args": {"name": "device"}},
                                    {"ph": "M", "pid": self.rank, "name": "process_name", "args": {"name": f"rank {self.rank}"}}]
        for s in self.spans:
            ev.append({"ph": "X", "pid": self.rank, "tid": 0, "name": s.name, "ts": s.start_us, "dur": s.host_us, "args": s.args})
            if s.device_us is not None:
                ev.append({"ph": "X", "pid": self.rank, "tid": 1, "name": s.name, "ts": s.start_us, "dur": s.device_us, "args": s.args})
        return ev

    def export(self, path: str) -> str:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path + ".tmp", "w") as f:
            json.dump({"traceEvents": self.events(), "displayTimeUnit": "ms"}, f)
        os.replace(path + ".tmp", path)
        return path

    def clear(self) -> None:
        self.spans.clear()
        self._pending.clear()
        self._t0 = self.clock()


def merge(paths: Sequence[str], out: str) -> str:
    """Join per-rank trace files into one (each keeps its own process id)."""
    events: List[Dict[str, Any]] = []
    for p in paths:
        with open(p) as f:
            events += json.load(f)["traceEvents"]
    with open(out, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
    return out


def breakdown(spans: Iterable[Span], collectives: Sequence[str] = ("all_reduce", "all_gather", "reduce_scatter", "all_to_all", "exchange"),
              wall_us: Optional[float] = None) -> Dict[str, float]:
    """Top-level spans' device time split into compute and collectives (by name), and the idle remainder of ``wall_us``."""
    top = [s for s in spans if s.depth == 0]
    comm = sum((s.device_us if s.device_us is not None else s.host_us) for s in top if any(c in s.name for c in collectives))
    total = sum((s.device_us if s.device_us is not None else s.host_us) for s in top)
    wall = wall_us if wall_us is not None else (max((s.start_us + s.host_us for s in top), default=0.0) - min((s.start_us for s in top), default=0.0))
    return {"compute_us": total - comm, "collective_us": comm, "idle_us": max(0.0, wall - total), "wall_us": wall}


TRACER = Tracer()          # the process's tracer: ``trace.TRACER.enabled = True`` around the steps to capture
