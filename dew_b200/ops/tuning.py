"""Measured kernel choices with a persistent cache.

``KernelOp`` names an operation with several candidate implementations; ``pick(case_key, candidates, run)`` times each
candidate on the device (CUDA events, warm-up, median), remembers the fastest under a key made of the op, the case and
the device, and persists the table as JSON so later processes skip the measurement.  Timing happens only when
``tune=True`` (or ``DEWB_TUNE=1``); otherwise a cached pick is used if present and the first candidate if not, so an
untuned run never pays for measurements.  ``record`` lets a benchmark write picks it measured itself.

Reference: src/dew/nn/kernels/tuning.py (``KernelOp`` autotune cache, 1693 lines), launches.py, tables.py.
"""
from __future__ import annotations

import json
import os
import statistics
import threading
from typing import Any, Callable, Dict, Hashable, Optional, Sequence

import torch

_LOCK = threading.Lock()
ENABLED: Optional[bool] = None          # set by ``enable``; None defers to the DEWB_TUNE environment variable


def enable(on: bool = True) -> None:
    """Let ``KernelOp.pick`` measure candidates it has no cached pick for (``Trainer(tune_kernels=True)`` calls this)."""
    global ENABLED
    ENABLED = bool(on)


def default_path() -> str:
    return os.environ.get("DEWB_TUNE_CACHE", os.path.join(os.path.expanduser("~"), ".cache", "dew_b200", "tuning.json"))


def device_key(device=None) -> str:
    if not torch.cuda.is_available():
        return "cpu"
    p = torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device())
    return f"{p.name}|sm{p.major}{p.minor}|{p.multi_processor_count}sm"


def time_once(fn: Callable[[], Any], iters: int = 5, warmup: int = 2) -> float:
    """Median milliseconds of ``fn`` on the current stream (CUDA events), or wall-clock on CPU."""
    for _ in range(warmup):
        fn()
    if not torch.cuda.is_available():
        import time
        ts = []
        for _ in range(iters):
            t0 = time.perf_counter(); fn(); ts.append((time.perf_counter() - t0) * 1e3)
        return statistics.median(ts)
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record(); b.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


class TuningCache:
    def __init__(self, path: Optional[str] = None):
        self.path = path or default_path()
        self.table: Dict[str, Dict[str, Any]] = {}
        self._loaded = False

    def _load(self) -> None:
        if self._loaded:
            return
        self._loaded = True
        try:
            with open(self.path) as f:
                self.table = json.load(f)
        except (OSError, ValueError):
            self.table = {}

    def get(self, key: str) -> Optional[Dict[str, Any]]:
        self._load()
        return self.table.get(key)

    def put(self, key: str, entry: Dict[str, Any]) -> None:
        with _LOCK:
            self._load()
            self.table[key] = entry
            try:
                os.makedirs(os.path.dirname(self.path) or ".", exist_ok=True)
                tmp = f"{self.path}.{os.getpid()}.tmp"
                with open(tmp, "w") as f:
                    json.dump(self.table, f, indent=1, sort_keys=True)
                os.replace(tmp, self.path)                  # atomic: readers never see a torn table
            except OSError:
                pass


CACHE = TuningCache()


class KernelOp:
    def __init__(self, name: str, cache: Optional[TuningCache] = None):
        self.name, self.cache = name, cache or CACHE
        self.picks: Dict[str, str] = {}                      # in-process memo

    def key(self, case: Hashable, device=None) -> str:
        return f"{self.name}|{case}|{device_key(device)}"

    def record(self, case: Hashable, choice: str, timings: Optional[Dict[str, float]] = None, device=None) -> None:
        k = self.key(case, device)
        self.picks[k] = choice
        self.cache.put(k, {"choice": choice, "ms": timings or {}})

    def pick(self, case: Hashable, candidates: Sequence[str], run: Optional[Callable[[str], Any]] = None,
             tune: Optional[bool] = None, device=None) -> str:
        """The candidate to use for ``case``.  ``run(name)`` executes one candidate (it may raise to refuse the case)."""
        k = self.key(case, device)
        if k in self.picks:
            return self.picks[k]
        hit = self.cache.get(k)
        if hit is not None and hit.get("choice") in candidates:
            self.picks[k] = hit["choice"]
            return hit["choice"]
        if tune is None:
            tune = ENABLED if ENABLED is not None else bool(int(os.environ.get("DEWB_TUNE", "0")))
        if not tune or run is None:
            return candidates[0]
        timings: Dict[str, float] = {}
        for name in candidates:
            try:
                timings[name] = time_once(lambda: run(name))
            except Exception:
                continue                                     # a refusing candidate is simply not a choice
        if not timings:
            return candidates[0]
        best = min(timings, key=timings.get)
        self.record(case, best, timings, device)
        return best
