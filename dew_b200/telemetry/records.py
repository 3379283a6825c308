"""Benchmark records: one JSON line per measurement, stamped with what it was measured on, appended atomically.

``stamp()`` gathers the environment a number belongs to (device name and SM count, driver / CUDA / torch versions, the repository's
commit when it is a git checkout, the host, the time); ``Records(path).append(record)`` writes ``{**stamp, **record}`` as one line;
``read`` / ``latest`` / ``compare`` read them back - ``compare`` lines two runs' records up by a key and reports the ratio of a field,
which the performance gate and the benchmark tables are built from.

Reference: src/dew/telemetry/records.py, src/dew/telemetry/export.py.
"""
from __future__ import annotations

import json
import os
import platform
import subprocess
import time
from typing import Any, Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch


def stamp(repository: Optional[str] = None) -> Dict[str, Any]:
    out: Dict[str, Any] = {"time": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "host": platform.node(), "torch": torch.__version__,
                           "cuda": torch.version.cuda}
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        out.update(device=p.name, sms=p.multi_processor_count, memory_gb=round(p.total_memory / 1e9, 1), devices=torch.cuda.device_count())
    else:
        out["device"] = "cpu"
    repo = repository or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        out["commit"] = subprocess.run(["git", "-C", repo, "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5).stdout.strip() or None
    except (OSError, subprocess.SubprocessError):
        out["commit"] = None
    return out


class Records:
    def __init__(self, path: str, stamp_fn: Callable[[], Mapping[str, Any]] = stamp):
        self.path, self._stamp = path, stamp_fn
        self._cached: Optional[Dict[str, Any]] = None

    def append(self, record: Mapping[str, Any]) -> Dict[str, Any]:
        if self._cached is None:
            self._cached = dict(self._stamp())
        row = {**self._cached, **record}
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        line = json.dumps(row, default=float) + "\n"
        with open(self.path, "a") as f:                                     # one write per line: appends of concurrent ranks do not interleave
            f.write(line)
        return row

    def read(self) -> List[Dict[str, Any]]:
        if not os.path.exists(self.path):
            return []
        with open(self.path) as f:
            return [json.loads(l) for l in f if l.strip()]

    def latest(self, **match) -> Optional[Dict[str, Any]]:
        rows = [r for r in self.read() if all(r.get(k) == v for k, v in match.items())]
        return rows[-1] if rows else None


def compare(before: Iterable[Mapping[str, Any]], after: Iterable[Mapping[str, Any]], key: Sequence[str], field: str) -> List[Dict[str, Any]]:
    """Records of two runs lined up by ``key`` fields: ``{key..., before, after, ratio}`` per key present in both (the last record of
    each key wins)."""
    index = lambda rows: {tuple(r.get(k) for k in key): r for r in rows if field in r}
    a, b = index(before), index(after)
    out = []
    for k in a:
        if k in b and a[k][field]:
            out.append({**dict(zip(key, k)), "before": a[k][field], "after": b[k][field], "ratio": b[k][field] / a[k][field]})
    return out
