"""``sample``: run the reverse process from ``x_T`` with a solver over a descending time grid.

Parity with src/dew/sampling/walks.py:53-227: exactly one of ``steps`` / ``times``; every step's noise comes
from ``key`` folded with the step index; optional ``record(x, state, denoised)`` stacked over steps;
``final_denoise`` returns the model's clean prediction at the last grid point.  The loop is a plain host
loop; on a GPU the per-step work is the model call, which dominates, and callers that want one launch
capture the whole walk in a CUDA graph (``dew_b200.inference``).
"""
from __future__ import annotations

from typing import Any, Callable, Optional, Sequence

import torch

from ..utils import keys as K


def sample(denoise, x_T: torch.Tensor, steps: Optional[int] = None, *, solver, guidance=None, key=0,
           times: Optional[Sequence[float]] = None, initial: Any = None, final_denoise: bool = True,
           record: Optional[Callable] = None, null_conditions=None):
    if (steps is None) == (times is None):
        raise ValueError("pass exactly one of steps and times")
    if steps is not None and (type(steps) is not int or steps < 1):
        raise ValueError("steps must be a positive integer")
    process = denoise.process
    key = K.key(key) if not isinstance(key, int) or key < (1 << 32) else key
    grid = process.times(steps) if times is None else torch.as_tensor(times, dtype=torch.float32)
    if grid.dim() != 1 or grid.shape[0] < 1:
        raise ValueError(f"times must be a descending grid of at least one point, got {tuple(grid.shape)}")
    if not bool(torch.isfinite(grid).all()) or bool((grid[1:] - grid[:-1] > 0).any()):
        raise ValueError("times must be a finite descending grid")
    call = guidance.wrap(denoise, null_conditions) if guidance is not None else denoise
    batch = x_T.shape[0]
    dev = x_T.device

    def full(t):
        return torch.full((batch,), float(t), device=dev, dtype=torch.float32)

    if grid.shape[0] == 1:
        if record is not None:
            raise ValueError("a record reads the steps, and a grid of one point takes none")
        return call(x_T, full(grid[0]))[0] if final_denoise else x_T
    state = solver.init(x_T, grid, process, key=key) if initial is None else initial
    x = x_T
    readings = []
    with torch.no_grad():
        for i in range(grid.shape[0] - 1):
            t, t_next = full(grid[i]), full(grid[i + 1])
            denoised, eps = call(x, t)
            x, state = solver.step(x, t, t_next, denoised, eps, state, K.fold_in(key, i), process, call)
            if record is not None:
                readings.append(record(x, state, denoised))
        if final_denoise and float(grid[-1]) > 0:
            x = call(x, full(grid[-1]))[0]
    if record is None:
        return x
    return x, readings


def walk_and_decode(denoise, x_T, steps=None, *, solver, autoencoder=None, clip=(-1.0, 1.0), **kw):
    x = sample(denoise, x_T, steps, solver=solver, **kw)
    if autoencoder is not None:
        x = autoencoder.decode(x)
    return x.clamp(*clip) if clip is not None else x
