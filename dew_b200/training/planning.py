"""Fit search: find the largest microbatch (and whether to rematerialise) that fits the device's memory, by running
trial steps down a ladder of plans.

A ``Plan`` is (microbatch rows, rematerialisation on / off).  ``FitSearch.run`` walks the ladder from the cheapest-to-run
plan (largest microbatch, no remat) towards the most frugal one, executes ``trial(plan)`` (one forward + backward on a
sample batch) and accepts the first plan whose peak memory stays under ``limit_fraction`` of the device; an
out-of-memory error is caught, the cache emptied, and the next rung tried.  On CPU (or when ``measure`` is supplied) the
memory of a trial comes from the callback, which is how the search is tested without a GPU.

Reference: src/dew/training/planning.py (``FitSearch`` and its remat ladder), src/dew/training/memory.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch


@dataclass(frozen=True)
class Plan:
    microbatch: int
    remat: bool = False

    def microbatches(self, rows: int) -> int:
        return rows // self.microbatch


class NoPlanFits(RuntimeError):
    pass


def ladder(rows: int, allow_remat: bool = True, min_microbatch: int = 1) -> List[Plan]:
    """Divisors of ``rows`` from the whole batch down, each first without and then with rematerialisation."""
    sizes = [m for m in range(rows, min_microbatch - 1, -1) if rows % m == 0]
    out: List[Plan] = []
    for m in sizes:
        out.append(Plan(m, False))
        if allow_remat:
            out.append(Plan(m, True))
    return out


@dataclass
class Trial:
    plan: Plan
    peak_bytes: Optional[int]
    fits: bool
    error: Optional[str] = None


class FitSearch:
    def __init__(self, rows: int, *, limit_fraction: float = 0.92, capacity_bytes: Optional[int] = None, allow_remat: bool = True,
                 measure: Optional[Callable[[Plan], int]] = None, device=None):
        self.rows, self.limit_fraction, self.allow_remat = rows, limit_fraction, allow_remat
        self.measure = measure
        self.device = device
        if capacity_bytes is None:
            if torch.cuda.is_available() and measure is None:
                capacity_bytes = torch.cuda.get_device_properties(device or 0).total_memory
            else:
                capacity_bytes = 1 << 62
        self.capacity = capacity_bytes
        self.trials: List[Trial] = []

    def _run_trial(self, plan: Plan, trial: Optional[Callable[[Plan], None]]) -> Trial:
        if self.measure is not None:
            peak = int(self.measure(plan))
            return Trial(plan, peak, peak <= self.limit_fraction * self.capacity)
        torch.cuda.reset_peak_memory_stats(self.device)
        try:
            trial(plan)
            torch.cuda.synchronize(self.device)
        except torch.cuda.OutOfMemoryError as e:
            torch.cuda.empty_cache()
            return Trial(plan, None, False, str(e)[:120])
        peak = torch.cuda.max_memory_allocated(self.device)
        return Trial(plan, peak, peak <= self.limit_fraction * self.capacity)

    def run(self, trial: Optional[Callable[[Plan], None]] = None, plans: Optional[Sequence[Plan]] = None, remembered: Optional["PlanRecords"] = None,
            key: Optional[str] = None) -> Plan:
        """``remembered`` / ``key``: plans chosen by earlier runs of the same step (same model, batch and device): the search starts at
        the rung an earlier run settled on instead of at the top of the ladder, and records where this one settles."""
        rungs = list(plans or ladder(self.rows, self.allow_remat))
        if remembered is not None and key is not None:
            earlier = remembered.get(key)
            if earlier is not None and earlier in rungs:
                rungs = rungs[rungs.index(earlier):]                      # a rung that did not fit before is not tried again
        for plan in rungs:
            t = self._run_trial(plan, trial)
            self.trials.append(t)
            if t.fits:
                if remembered is not None and key is not None:
                    remembered.put(key, plan, t.peak_bytes)
                return plan
        raise NoPlanFits(f"no plan fits {self.limit_fraction:.0%} of {self.capacity / 2**30:.1f} GiB: " +
                         ", ".join(f"{t.plan.microbatch}{'r' if t.plan.remat else ''}" for t in self.trials))

    def report(self) -> str:
        rows = [f"{'microbatch':>10} {'remat':>5} {'peak GiB':>9} fits"]
        for t in self.trials:
            peak = "oom" if t.peak_bytes is None else f"{t.peak_bytes / 2**30:.2f}"
            rows.append(f"{t.plan.microbatch:>10} {str(t.plan.remat):>5} {peak:>9} {t.fits}")
        return "\n".join(rows)


class PlanRecords:
    """The plan each step settled on, kept in a JSON file beside a run's caches, keyed by a digest of what determines the step's
    memory (``step_key``): a later run of the same step starts its search there, as a resumed run starts at its checkpoint."""

    def __init__(self, path: str):
        self.path = path

    def _read(self) -> dict:
        import json
        import os
        if not os.path.exists(self.path):
            return {}
        try:
            with open(self.path) as f:
                return json.load(f)
        except (OSError, ValueError):
            return {}

    def get(self, key: str) -> Optional[Plan]:
        rec = self._read().get(key)
        return None if rec is None else Plan(int(rec["microbatch"]), bool(rec["remat"]))

    def put(self, key: str, plan: Plan, peak_bytes: Optional[int] = None) -> None:
        import json
        import os
        data = self._read()
        data[key] = {"microbatch": plan.microbatch, "remat": plan.remat, "peak_bytes": peak_bytes}
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        with open(self.path + ".tmp", "w") as f:
            json.dump(data, f, indent=1)
        os.replace(self.path + ".tmp", self.path)


def step_key(model: torch.nn.Module, batch_shape: Sequence[int], dtype: str = "bfloat16", device: Optional[str] = None, extra: str = "") -> str:
    """A digest of what a step's memory depends on: the parameters' names, shapes and dtypes, the batch's shape, the compute dtype
    and the device."""
    import hashlib
    h = hashlib.sha256()
    for n, p in model.named_parameters():
        h.update(f"{n}:{tuple(p.shape)}:{p.dtype};".encode())
    if device is None:
        device = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    h.update(f"|{tuple(batch_shape)}|{dtype}|{device}|{extra}".encode())
    return h.hexdigest()[:20]
