"""FLOP and memory accounting of a training step, and model-FLOP utilisation.

There is no compiled program to read the cost from, so the FLOPs of a step are *counted*: the objective's loss and its
backward run once under ``torch.utils.flop_counter.FlopCounterMode`` on CPU tensors (where every op of this library takes
its PyTorch form, whose matmuls, convolutions and attention the counter knows), which gives forward and backward FLOPs per
operator family for any model or objective - the analogue of reading them off the compiled step.  Memory comes from the
caching allocator's statistics plus, for the sharded engines, their own state breakdown.

Reference: src/dew/telemetry/instrumentation.py (``StepFlops`` :1018, ``step_flops`` :1120, ``compiled_memory`` :1104,
``model_flops_utilization`` :1196).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional

import torch


@dataclass(frozen=True)
class StepFlops:
    forward: float
    backward: float
    by_operator: Dict[str, float] = field(default_factory=dict)

    @property
    def total(self) -> float:
        return self.forward + self.backward


def step_flops(objective, batch: Mapping[str, torch.Tensor], rows: Optional[int] = None) -> StepFlops:
    """FLOPs of one loss + backward of ``objective`` on ``batch`` (counted on a CPU copy of the model; pass ``rows`` to count
    on the first rows only and scale - FLOPs are linear in the batch)."""
    from torch.utils.flop_counter import FlopCounterMode
    from ..objectives.base import Step
    model = objective.model
    cpu_model = copy.deepcopy(model).to("cpu").float()
    obj = copy.copy(objective)
    obj.model = cpu_model
    n = next(iter(batch.values())).shape[0]
    take = min(n, rows) if rows else n
    small = {k: (v[:take].cpu() if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
    scale = n / take

    def run(with_backward: bool):
        with FlopCounterMode(display=False) as counter:
            out = obj.loss(None, small, Step(step=0, key=0, train=True, device=torch.device("cpu")))
            stats = out[0] if isinstance(out, tuple) else out
            total, _ = obj.reduce_loss(stats)
            if with_backward:
                total.backward()
        per = {}
        for op, f in counter.get_flop_counts().get("Global", {}).items():
            per[str(op)] = per.get(str(op), 0.0) + float(f)
        return float(counter.get_total_flops()), per
    fwd, _ = run(False)
    both, per = run(True)
    return StepFlops(fwd * scale, (both - fwd) * scale, {k: v * scale for k, v in per.items()})


def memory_report(device: Optional[torch.device] = None, engine: Any = None) -> Dict[str, float]:
    """Bytes now / at peak from the caching allocator (GPU) plus the engine's own breakdown of parameter / gradient /
    optimizer state where it offers one."""
    out: Dict[str, float] = {}
    if torch.cuda.is_available():
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        s = torch.cuda.memory_stats(dev)
        out.update(allocated=float(s.get("allocated_bytes.all.current", 0)), peak=float(s.get("allocated_bytes.all.peak", 0)),
                   reserved=float(s.get("reserved_bytes.all.current", 0)))
    if engine is not None and hasattr(engine, "state_bytes"):
        out.update({f"state/{k}": float(v) for k, v in engine.state_bytes().items()})
    return out


def model_flops_utilization(flops_per_step: float, ms_per_step: float, devices: int = 1, peak_tflops: Optional[float] = None) -> float:
    """Achieved FLOP/s over the peak of ``devices`` GPUs (datasheet dense bf16 2250 TFLOP/s unless ``peak_tflops`` is given)."""
    peak = (peak_tflops if peak_tflops is not None else 2250.0) * 1e12 * devices
    return flops_per_step / (ms_per_step * 1e-3) / peak
