"""Performance gate: compare benchmark records (the JSON lines ``bench.py`` / the kernel benchmarks print) with a committed
gate file and fail when a number regressed beyond its tolerance.

    python -m dew_b200.telemetry.perf_gate --records BENCH.json --gate gates.json

A gate file maps a record selector to bounds::

    {"gates": [{"match": {"metric": "train tokens/sec (dense 8B LM, FSDP)", "n_gpus": 1}, "field": "value", "min": 20000, "tolerance": 0.03},
               {"match": {"kernel": "gemm_sm100", "name": "fwd qkv"}, "field": "pair_ms", "max": 0.30}]}

``min`` / ``max`` are the accepted bounds; ``tolerance`` widens them by that fraction (measurement noise).  A gate with no
matching record fails too unless ``"optional": true``.  Reference: tools/perf_gate.py.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Any, Dict, Iterable, List, Mapping, Tuple


def read_records(path: str) -> List[Dict[str, Any]]:
    text = open(path).read().strip()
    if not text:
        return []
    try:
        data = json.loads(text)
        if isinstance(data, dict):
            # a driver record wraps the line it captured: look for embedded JSON lines in its string values too
            out = [data]
            for v in _strings(data):
                out += [json.loads(l) for l in v.splitlines() if l.startswith("{") and l.rstrip().endswith("}") and _is_json(l)]
            return out
        return list(data)
    except ValueError:
        return [json.loads(l) for l in text.splitlines() if l.startswith("{") and _is_json(l)]


def _is_json(line: str) -> bool:
    try:
        json.loads(line)
        return True
    except ValueError:
        return False


def _strings(d: Any) -> Iterable[str]:
    if isinstance(d, str):
        yield d
    elif isinstance(d, Mapping):
        for v in d.values():
            yield from _strings(v)
    elif isinstance(d, (list, tuple)):
        for v in d:
            yield from _strings(v)


def _field(record: Mapping[str, Any], path: str) -> Any:
    cur: Any = record
    for part in path.split("."):
        if not isinstance(cur, Mapping) or part not in cur:
            return None
        cur = cur[part]
    return cur


def check(records: List[Mapping[str, Any]], gates: List[Mapping[str, Any]]) -> Tuple[bool, List[str]]:
    ok, lines = True, []
    for g in gates:
        hits = [r for r in records if all(_field(r, k) == v for k, v in g["match"].items())]
        if not hits:
            if not g.get("optional"):
                ok = False
                lines.append(f"FAIL  no record matches {g['match']}")
            continue
        tol = float(g.get("tolerance", 0.0))
        for r in hits:
            v = _field(r, g["field"])
            if v is None:
                ok = False
                lines.append(f"FAIL  {g['match']}: record has no field {g['field']!r}")
                continue
            bad = ("min" in g and v < g["min"] * (1 - tol)) or ("max" in g and v > g["max"] * (1 + tol))
            ok = ok and not bad
            bound = " ".join(f"{k} {g[k]}" for k in ("min", "max") if k in g)
            lines.append(f"{'FAIL' if bad else 'ok  '}  {g['match']}: {g['field']} = {v:.6g} ({bound}, tolerance {tol:.0%})")
    return ok, lines


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--records", required=True, action="append")
    ap.add_argument("--gate", required=True)
    args = ap.parse_args(argv)
    records: List[Dict[str, Any]] = []
    for p in args.records:
        records += read_records(p)
    gates = json.load(open(args.gate))["gates"]
    ok, lines = check(records, gates)
    print("\n".join(lines))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
