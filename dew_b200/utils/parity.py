"""The accuracy contract as a function: an implementation is *on par* with a reference where its error from the float64
truth is within ``PARITY`` times the reference's on the same inputs, judged over drawn seeds.

For every seed the caller's three arms run on the same inputs: ``truth`` (float64), ``reference`` (e.g. PyTorch in bf16)
and ``candidate`` (e.g. a CUDA kernel).  Each leaf of the outputs records two errors per seed: the RMS error from the
truth, and the worst row's RMS error (an RMS over every entry averages a few wrong rows away, so the worst row is held to
``ROW_FACTOR`` times the reference's worst row).  The pooled ratio is sqrt(sum cand^2 / sum ref^2) over seeds; its
interval is a percentile bootstrap over the seeds (``BOOTSTRAP`` resamples from one fixed key, so a check decides alike on
every run).  A leaf passes when the interval's upper end is within ``PARITY``, is *over* when its lower end is above it,
and is inconclusive otherwise or with fewer than ``FEWEST_SEEDS`` seeds.

Reference: src/dew/parity.py (``PARITY`` 1.5, ``ROW_FACTOR`` 4, ``BOOTSTRAP`` 2000, ``FEWEST_SEEDS`` 8, ``Finding``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping, Sequence

import torch

PARITY = 1.5
ROW_FACTOR = 4.0
BOOTSTRAP = 2000
LOWER_TAIL, UPPER_TAIL = 5e-4, 5e-4
FEWEST_SEEDS = 8


@dataclass(frozen=True)
class Finding:
    leaf: str
    status: str            # "pass" | "over" | "inconclusive" | "rows_over" | "not_finite" | "exact"
    ratio: float           # pooled RMS ratio candidate / reference (inf when the reference is exact and the candidate is not)
    low: float
    high: float
    worst_row_ratio: float
    seeds: int

    @property
    def ok(self) -> bool:
        return self.status in ("pass", "exact")


def _leaves(out: Any, prefix: str = "") -> Dict[str, torch.Tensor]:
    if isinstance(out, torch.Tensor):
        return {prefix or "out": out}
    if isinstance(out, Mapping):
        flat: Dict[str, torch.Tensor] = {}
        for k, v in out.items():
            flat.update(_leaves(v, f"{prefix}.{k}" if prefix else str(k)))
        return flat
    if isinstance(out, (tuple, list)):
        flat = {}
        for i, v in enumerate(out):
            flat.update(_leaves(v, f"{prefix}[{i}]" if prefix else f"[{i}]"))
        return flat
    raise TypeError(f"an arm returns tensors, mappings or sequences of them, not {type(out).__name__}")


def _errors(x: torch.Tensor, truth: torch.Tensor):
    """(sum of squared error, entries, worst row's mean squared error) against the float64 truth."""
    d = (x.detach().double().cpu() - truth.detach().double().cpu())
    rows = d.reshape(-1, d.shape[-1]) if d.dim() > 1 else d.reshape(1, -1)
    return float((d * d).sum()), d.numel(), float((rows * rows).mean(1).max())


def assess(candidate: Callable[[int], Any], reference: Callable[[int], Any], truth: Callable[[int], Any], seeds: Sequence[int],
           *, parity: float = PARITY, row_factor: float = ROW_FACTOR) -> List[Finding]:
    """Run the three arms on every seed and judge every output leaf.  Each arm maps a seed to its outputs (it draws its own
    inputs from the seed, so all three see the same ones)."""
    per: Dict[str, List[tuple]] = {}
    for seed in seeds:
        t, r, c = _leaves(truth(seed)), _leaves(reference(seed)), _leaves(candidate(seed))
        if set(t) != set(r) or set(t) != set(c):
            raise ValueError(f"the arms return different leaves: {sorted(t)} / {sorted(r)} / {sorted(c)}")
        for name in t:
            finite = bool(torch.isfinite(c[name].detach().float()).all())
            per.setdefault(name, []).append((_errors(c[name], t[name]), _errors(r[name], t[name]), finite))
    g = torch.Generator().manual_seed(0x5EED)
    findings = []
    for name, rec in per.items():
        n = len(rec)
        cs = torch.tensor([e[0][0] for e in rec], dtype=torch.float64)
        rs = torch.tensor([e[1][0] for e in rec], dtype=torch.float64)
        cw, rw = max(e[0][2] for e in rec), max(e[1][2] for e in rec)
        row_ratio = math.sqrt(cw / rw) if rw > 0 else (0.0 if cw == 0 else math.inf)
        if not all(e[2] for e in rec):
            findings.append(Finding(name, "not_finite", math.inf, math.inf, math.inf, row_ratio, n))
            continue
        if float(rs.sum()) == 0.0:
            exact = float(cs.sum()) == 0.0
            findings.append(Finding(name, "exact" if exact else "over", 0.0 if exact else math.inf, 0.0, 0.0 if exact else math.inf, row_ratio, n))
            continue
        ratio = math.sqrt(float(cs.sum() / rs.sum()))
        idx = torch.randint(0, n, (BOOTSTRAP, n), generator=g)
        boot = torch.sqrt(cs[idx].sum(1) / rs[idx].sum(1).clamp_min(1e-300))
        low, high = float(torch.quantile(boot, LOWER_TAIL)), float(torch.quantile(boot, 1 - UPPER_TAIL))
        if row_ratio > row_factor:
            status = "rows_over"
        elif n < FEWEST_SEEDS:
            status = "inconclusive"
        elif high <= parity:
            status = "pass"
        elif low > parity:
            status = "over"
        else:
            status = "inconclusive"
        findings.append(Finding(name, status, ratio, low, high, row_ratio, n))
    return findings


def assert_on_par(candidate, reference, truth, seeds: Sequence[int] = tuple(range(FEWEST_SEEDS)), **kw) -> List[Finding]:
    """``assess`` and raise ``AssertionError`` naming every leaf that is not on par."""
    findings = assess(candidate, reference, truth, seeds, **kw)
    bad = [f for f in findings if not f.ok]
    if bad:
        raise AssertionError("; ".join(f"{f.leaf}: {f.status} (ratio {f.ratio:.3g} in [{f.low:.3g}, {f.high:.3g}], worst row "
                                       f"{f.worst_row_ratio:.3g}x, {f.seeds} seeds)" for f in bad))
    return findings
