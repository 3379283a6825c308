"""``Profiler`` and ``region``: NVTX-named regions and torch.profiler captures, process-local, inert when idle.

Parity: src/dew/telemetry/profile.py (``CaptureOptions`` :110, ``Profiler`` :300-512, ``region`` :567) and
src/dew/telemetry/trace.py (device compute vs collectives vs idle from a capture).
"""
from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass
from typing import Dict, Optional

import torch


@dataclass(frozen=True)
class CaptureOptions:
    directory: Optional[str] = None
    cpu: bool = True
    cuda: bool = True
    record_shapes: bool = False
    with_stack: bool = False


@contextlib.contextmanager
def region(name: str):
    """An NVTX range on the GPU timeline (a no-op without CUDA)."""
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if cuda:
            torch.cuda.nvtx.range_pop()


class Profiler:
    def __init__(self, options: CaptureOptions = CaptureOptions()):
        self.options = options
        self._prof = None
        self.report: Optional[Dict[str, float]] = None

    def start(self) -> None:
        acts = [torch.profiler.ProfilerActivity.CPU] if self.options.cpu else []
        if self.options.cuda and torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts, record_shapes=self.options.record_shapes, with_stack=self.options.with_stack)
        self._prof.__enter__()

    def stop(self) -> Dict[str, float]:
        self._prof.__exit__(None, None, None)
        avgs = self._prof.key_averages()
        total = comm = 0.0
        for e in avgs:
            t = getattr(e, "self_device_time_total", 0.0) or 0.0
            total += t
            if any(s in e.key.lower() for s in ("nccl", "rs_adamw_ag", "allreduce_rows", "allgather_pull")):
                comm += t
        self.report = {"device_us": total, "collective_us": comm, "compute_us": total - comm}
        if self.options.directory:
            os.makedirs(self.options.directory, exist_ok=True)
            self._prof.export_chrome_trace(os.path.join(self.options.directory, "trace.json"))
        self.table = avgs.table(sort_by="self_cpu_time_total", row_limit=30)
        self._prof = None
        return self.report

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()
