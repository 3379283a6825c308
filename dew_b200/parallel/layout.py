"""``Layout``: rules mapping the logical axes declared on parameters to mesh axes, and the dry-run placement report.

Parity: src/dew/mesh.py:101-146 (``DEFAULT_RULES``: ``mlp / heads / kv / vocab -> tensor``, leading dimension of
every leaf >= ``min_shard`` elements ``-> fsdp``, ``experts -> expert``, residual width whole), ``logical_spec`` :162-218,
src/dew/distributed/placement.py:406-874 (``Layout`` fields, ``check`` / ``validate``, implied collectives, bytes per
device), ``LayoutRefused`` (mesh.py:46).  ``placement_report`` runs on the host for a *target* device count and memory
size without allocating on any device (``Trainer.validate``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .mesh import LayoutRefused, MeshSpec

DEFAULT_RULES: Tuple[Tuple[str, Optional[str]], ...] = (
    ("mlp", "tensor"), ("heads", "tensor"), ("kv", "tensor"), ("vocab", "tensor"), ("experts", "expert"),
    ("embed", None), ("norm", None), ("modulation", None), ("patch", None),
)


@dataclass(frozen=True)
class Layout:
    rules: Tuple[Tuple[str, Optional[str]], ...] = DEFAULT_RULES
    min_shard: int = 2 ** 16           # leaves smaller than this stay whole on the fsdp axis
    tolerance: float = 0.02            # accepted imbalance of bytes per device
    host: Tuple[str, ...] = ()         # state kinds kept in pinned host memory ("opt_state", "ema")
    host_parameters: Tuple[str, ...] = ()
    frozen_whole: bool = False
    stage_local: bool = True
    data_axes: Tuple[str, ...] = ()
    # "resident": every rank keeps a gathered compute copy of the parameters and full fp32 gradient accumulators (fastest while
    # they fit); "sharded": parameters and gradients live as shards and are gathered / reduced unit by unit (ZeRO-3);
    # "auto": resident when its unsharded state fits in `memory_fraction` of the device, else sharded
    memory: str = "auto"
    memory_fraction: float = 0.45

    def axis_for(self, logical: Optional[str]) -> Optional[str]:
        for name, mesh_axis in self.rules:
            if name == logical:
                return mesh_axis
        return None

    def leaf_spec(self, shape: Sequence[int], logical_axes: Sequence[Optional[str]], sizes: Mapping[str, int]) -> Tuple[Optional[str], ...]:
        """Mesh axis (or None) per dimension of a leaf. Tensor / expert axes follow the rules; the fsdp axis shards the
        leading dimension when the leaf is large enough and that dimension divides."""
        spec: List[Optional[str]] = [None] * len(shape)
        for i, la in enumerate(logical_axes[: len(shape)]):
            ax = self.axis_for(la)
            if ax is not None and sizes.get(ax, 1) > 1 and shape[i] % sizes[ax] == 0:
                spec[i] = ax
        numel = 1
        for s in shape:
            numel *= s
        f = sizes.get("fsdp", 1)
        if f > 1 and numel >= self.min_shard and len(shape) > 0:
            lead = shape[0] // (sizes.get(spec[0], 1) if spec[0] else 1)
            if lead % f == 0:
                spec[0] = "fsdp" if spec[0] is None else f"{spec[0]}+fsdp"
        return tuple(spec)

    def check(self, module: torch.nn.Module, mesh: MeshSpec, devices: int) -> List[str]:
        """Reasons this layout cannot be placed (empty = fine)."""
        sizes = mesh.sizes(devices)
        problems = []
        for name, p in module.named_parameters():
            axes = getattr(p, "logical_axes", (None,) * p.dim())
            for i, la in enumerate(axes[: p.dim()]):
                ax = self.axis_for(la)
                if ax is not None and sizes.get(ax, 1) > 1 and p.shape[i] % sizes[ax]:
                    problems.append(f"{name}: dimension {i} ({la}={p.shape[i]}) does not divide by {ax}={sizes[ax]}")
        return problems


def _shard_factor(spec: Sequence[Optional[str]], sizes: Mapping[str, int]) -> int:
    f = 1
    for s in spec:
        if s:
            for a in s.split("+"):
                f *= sizes.get(a, 1)
    return f


def placement_report(module: torch.nn.Module, mesh: Optional[MeshSpec], layout: Layout, devices: int = 1,
                     memory_bytes: float = 180e9, state_dtype: str = "float32", ema: bool = False,
                     compute_bytes: int = 2) -> Dict[str, Any]:
    """Bytes per device (parameters in compute dtype, fp32 masters, optimizer moments, EMA, fp32 gradient accumulators),
    implied collectives per step, and refusal reasons - computed from shapes only."""
    mesh = mesh or MeshSpec()
    sizes = mesh.sizes(devices)
    problems = layout.check(module, mesh, devices)
    state_b = 4 if state_dtype == "float32" else 2
    per_leaf = []
    totals = {"compute": 0.0, "master": 0.0, "moments": 0.0, "ema": 0.0, "grads": 0.0}
    gathered = 0.0
    for name, p in module.named_parameters():
        axes = getattr(p, "logical_axes", (None,) * p.dim())
        spec = layout.leaf_spec(tuple(p.shape), axes, sizes)
        f = _shard_factor(spec, sizes)
        tp_only = 1
        for s in spec:
            if s:
                for a in s.split("+"):
                    if a != "fsdp":
                        tp_only *= sizes.get(a, 1)
        n = p.numel()
        # the gathered bf16 copy and the fp32 gradient accumulator are full along fsdp, sharded along tensor / expert
        totals["compute"] += n / tp_only * compute_bytes
        totals["grads"] += n / tp_only * 4
        totals["master"] += n / f * 4
        totals["moments"] += n / f * 2 * state_b
        totals["ema"] += (n / f * 4) if ema else 0.0
        gathered += n / tp_only * compute_bytes
        per_leaf.append({"name": name, "shape": tuple(p.shape), "spec": spec, "shard_factor": f})
    total = sum(totals.values())
    collectives = []
    if sizes["fsdp"] > 1 or sizes["data"] > 1:
        collectives.append({"kind": "reduce_scatter+adamw+all_gather (fused, per unit)", "axis": "fsdp/data",
                            "bytes_per_step_per_device": totals["grads"] * (1 - 1 / max(1, sizes["fsdp"] * sizes["data"])) + gathered})
    if sizes["tensor"] > 1:
        collectives.append({"kind": "all_reduce+residual+rmsnorm (fused), 2 per layer", "axis": "tensor"})
    if sizes["expert"] > 1:
        collectives.append({"kind": "token dispatch / combine (peer push / pull), 2 per sparse layer", "axis": "expert"})
    if sizes["stage"] > 1:
        collectives.append({"kind": "pipeline send / recv (NCCL p2p)", "axis": "stage"})
    if total > memory_bytes:
        problems.append(f"state needs {total / 1e9:.1f} GB per device, the device has {memory_bytes / 1e9:.0f} GB "
                        f"(activations not counted)")
    return {"devices": devices, "mesh": sizes, "bytes_per_device": totals, "total_bytes_per_device": total,
            "fits": total <= memory_bytes, "collectives": collectives, "refusals": problems, "leaves": per_leaf}
