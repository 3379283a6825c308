"""Trackers: where metrics and artifacts go.  ``LocalTracker`` writes JSONL + artifacts to disk; W&B / MLflow /
TensorBoard trackers bind their packages only when constructed *and* used (constructing opens nothing);
``Trackers`` fans out.  Parity: src/dew/training/tracker.py:59-811.
"""
from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Protocol, Sequence

import torch


def _scalar(v: Any) -> Any:
    if hasattr(v, "value") and callable(v.value):
        v = v.value()
    if isinstance(v, torch.Tensor):
        return float(v.detach().float().cpu()) if v.numel() == 1 else v.detach().float().cpu().tolist()
    return v


class Tracker(Protocol):
    def log(self, step: int, metrics: Mapping[str, Any]) -> None: ...
    def artifact(self, step: int, name: str, value: Any) -> None: ...
    def close(self) -> None: ...


class LocalTracker:
    def __init__(self, directory: os.PathLike, name: str = "run"):
        self.directory, self.name = Path(directory), name
        self._file = None

    def _open(self):
        if self._file is None:
            self.directory.mkdir(parents=True, exist_ok=True)
            self._file = open(self.directory / f"{self.name}.jsonl", "a", buffering=1)
        return self._file

    def log(self, step: int, metrics: Mapping[str, Any]) -> None:
        row = {"step": int(step), "time": time.time(), **{k: _scalar(v) for k, v in metrics.items()}}
        self._open().write(json.dumps(row) + "\n")

    def artifact(self, step: int, name: str, value: Any) -> None:
        d = self.directory / "artifacts" / f"{int(step):08d}"
        d.mkdir(parents=True, exist_ok=True)
        if hasattr(value, "save"):
            value.save(d / f"{name}.ppm")
        elif hasattr(value, "rows"):
            (d / f"{name}.json").write_text(json.dumps(value.rows(), indent=1))
        else:
            torch.save(value, d / f"{name}.pt")

    def history(self):
        path = self.directory / f"{self.name}.jsonl"
        return [json.loads(l) for l in path.read_text().splitlines()] if path.exists() else []

    def close(self) -> None:
        if self._file is not None:
            self._file.close()
            self._file = None


class MemoryTracker:
    """Keeps rows in memory (tests, notebooks)."""

    def __init__(self):
        self.rows, self.artifacts = [], []

    def log(self, step, metrics):
        self.rows.append({"step": int(step), **{k: _scalar(v) for k, v in metrics.items()}})

    def artifact(self, step, name, value):
        self.artifacts.append((int(step), name, value))

    def close(self):
        pass


class _Lazy:
    package = ""

    def _module(self):
        import importlib
        try:
            return importlib.import_module(self.package)
        except ImportError as e:
            raise ImportError(f"{type(self).__name__} needs the `{self.package}` package, which is not installed") from e


class WandbTracker(_Lazy):
    package = "wandb"

    def __init__(self, project: str, name: Optional[str] = None, config: Optional[dict] = None, **kw):
        self.project, self.name, self.config, self.kw, self._run = project, name, config, kw, None

    def _ensure(self):
        if self._run is None:
            self._run = self._module().init(project=self.project, name=self.name, config=self.config, **self.kw)
        return self._run

    def log(self, step, metrics):
        self._ensure().log({k: _scalar(v) for k, v in metrics.items()}, step=int(step))

    def artifact(self, step, name, value):
        wandb = self._module()
        if hasattr(value, "grid"):
            self._ensure().log({name: wandb.Image(value.grid().numpy())}, step=int(step))

    def close(self):
        if self._run is not None:
            self._run.finish()


Wandb = WandbTracker


class MLflowTracker(_Lazy):
    package = "mlflow"

    def __init__(self, experiment: str, run_name: Optional[str] = None):
        self.experiment, self.run_name, self._started = experiment, run_name, False

    def _ensure(self):
        m = self._module()
        if not self._started:
            m.set_experiment(self.experiment)
            m.start_run(run_name=self.run_name)
            self._started = True
        return m

    def log(self, step, metrics):
        self._ensure().log_metrics({k: float(_scalar(v)) for k, v in metrics.items()}, step=int(step))

    def artifact(self, step, name, value):
        pass

    def close(self):
        if self._started:
            self._module().end_run()


class TensorBoardTracker:
    def __init__(self, directory: os.PathLike):
        self.directory, self._writer = str(directory), None

    def _ensure(self):
        if self._writer is None:
            from torch.utils.tensorboard import SummaryWriter
            self._writer = SummaryWriter(self.directory)
        return self._writer

    def log(self, step, metrics):
        w = self._ensure()
        for k, v in metrics.items():
            s = _scalar(v)
            if isinstance(s, (int, float)):
                w.add_scalar(k, s, int(step))

    def artifact(self, step, name, value):
        if hasattr(value, "grid"):
            self._ensure().add_image(name, value.grid().permute(2, 0, 1), int(step))

    def close(self):
        if self._writer is not None:
            self._writer.close()


class ConsoleTracker:
    """One compact line per logged step on a stream: the step (of ``steps`` when known), the chosen scalars, the rate of the
    ``rate_key`` metric per second since the previous line, and an estimate of the time left.
    Reference: src/dew/training/display.py (the run's console display)."""

    def __init__(self, steps: Optional[int] = None, keys: Sequence[str] = ("loss", "learning_rate", "grad_norm"), rate_key: str = "tokens",
                 stream=None, clock=time.monotonic):
        import sys
        self.steps, self.keys, self.rate_key = steps, tuple(keys), rate_key
        self.stream = stream if stream is not None else sys.stderr
        self.clock = clock
        self._last = None               # (time, step)
        self._first = None

    @staticmethod
    def _fmt(v) -> str:
        if isinstance(v, float):
            return f"{v:.3e}" if (abs(v) < 1e-3 or abs(v) >= 1e4) and v != 0 else f"{v:.4f}"
        return str(v)

    @staticmethod
    def _span(seconds: float) -> str:
        s = int(max(seconds, 0))
        return f"{s // 3600}:{s % 3600 // 60:02d}:{s % 60:02d}"

    def log(self, step: int, metrics: Mapping[str, Any]) -> None:
        now = self.clock()
        row = {k: _scalar(v) for k, v in metrics.items()}
        parts = [f"step {int(step)}" + (f"/{self.steps}" if self.steps else "")]
        parts += [f"{k} {self._fmt(row[k])}" for k in self.keys if k in row and row[k] is not None]
        if self._last is not None and now > self._last[0]:
            dt, dsteps = now - self._last[0], int(step) - self._last[1]
            if self.rate_key in row and isinstance(row[self.rate_key], (int, float)) and dsteps > 0:
                parts.append(f"{row[self.rate_key] * dsteps / dt:,.0f} {self.rate_key}/s")
            parts.append(f"{dt / max(dsteps, 1):.3f} s/step")
        if self._first is None:
            self._first = (now, int(step))
        elif self.steps and int(step) > self._first[1]:
            per = (now - self._first[0]) / (int(step) - self._first[1])
            parts.append(f"eta {self._span(per * (self.steps - int(step)))}")
        self._last = (now, int(step))
        print(" | ".join(parts), file=self.stream, flush=True)

    def artifact(self, step: int, name: str, value: Any) -> None:
        print(f"step {int(step)} | artifact {name}: {type(value).__name__}", file=self.stream, flush=True)

    def close(self) -> None:
        pass


class Trackers:
    def __init__(self, *trackers):
        self.trackers = list(trackers)

    def log(self, step, metrics):
        for t in self.trackers:
            t.log(step, metrics)

    def artifact(self, step, name, value):
        for t in self.trackers:
            t.artifact(step, name, value)

    def close(self):
        for t in self.trackers:
            t.close()
