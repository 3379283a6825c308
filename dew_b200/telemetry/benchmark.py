"""Device timing with CUDA events, L2 eviction between samples, and roofline fractions against measured peaks.

Parity (capabilities): src/dew/telemetry/benchmark.py (``Benchmark`` :41, ``DeviceTime`` :295, L2 eviction :207-236,
paired ``compared`` :587).  Timing rules: warm-up first, a buffer larger than L2 written between timed iterations,
events on the launching stream with a synchronize on both sides; multi-GPU numbers are the max over ranks.
"""
from __future__ import annotations

import json
import os
import statistics
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, List, Optional

import torch

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measured_peaks() -> Dict[str, float]:
    """Copy bandwidth and cuBLAS bf16 throughput measured on this pool (``MEASURED_PEAKS.json`` at the repository
    root when present, else the stated fallback)."""
    for root in (Path(__file__).resolve().parents[2], Path.cwd()):
        p = root / "MEASURED_PEAKS.json"
        if p.exists():
            d = json.loads(p.read_text())
            d["source"] = "measured"
            return d
    return dict(FALLBACK_PEAKS)


class L2Flush:
    def __init__(self, device="cuda", nbytes: int = 2 * L2_BYTES):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def __call__(self):
        self.buf.fill_(1)


@dataclass
class DeviceTime:
    samples_ms: List[float]

    @property
    def median_ms(self) -> float:
        return statistics.median(self.samples_ms)

    @property
    def min_ms(self) -> float:
        return min(self.samples_ms)


def device_time(fn: Callable[[], None], warmup: int = 3, iters: int = 10, flush: Optional[L2Flush] = None,
                graph: bool = False) -> DeviceTime:
    """Median-able device time of ``fn``.  ``graph=True`` captures ``fn`` into a CUDA graph first and times replays, so
    host launch overhead (which dominates kernels of a few tens of microseconds) is excluded."""
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
            with torch.cuda.graph(g, stream=side):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        run = g.replay
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        fn = run
    out = []
    for _ in range(iters):
        if flush is not None:
            flush()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        out.append(s.elapsed_time(e))
    return DeviceTime(out)


def max_over_ranks(value: float) -> float:
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([value], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return value


def compared(a: Callable[[], None], b: Callable[[], None], pairs: int = 10, flush: Optional[L2Flush] = None) -> Dict[str, float]:
    """Paired A/B timing (alternating order) with a sign-test count, so clock drift hits both arms alike."""
    for _ in range(3):
        a(); b()
    wins = 0
    ta, tb = [], []
    for i in range(pairs):
        first, second = (a, b) if i % 2 == 0 else (b, a)
        x = device_time(first, warmup=0, iters=1, flush=flush).samples_ms[0]
        y = device_time(second, warmup=0, iters=1, flush=flush).samples_ms[0]
        xa, xb = (x, y) if i % 2 == 0 else (y, x)
        ta.append(xa); tb.append(xb)
        wins += xa < xb
    return {"a_ms": statistics.median(ta), "b_ms": statistics.median(tb), "a_wins": wins, "pairs": pairs}
