"""From a ``MeshSpec`` to a running engine: the mesh's axes are turned into process groups and the model, the optimizer
state and the step are arranged over them, so ``Trainer(mesh=MeshSpec(fsdp=4, tensor=2))`` needs no hand assembly.

What each axis does here (reference: ``MeshSpec`` and its placement, src/dew/distributed/placement.py:142-254,274-315; the
logical rules ``mlp / heads / kv / vocab -> tensor``, ``experts -> expert``, leading dimension ``-> fsdp``,
src/dew/mesh.py:101-146; stage-local optimizer state, src/dew/training/stages.py):

``tensor``    the model is split Megatron-style in place (``parallel.tp.tensor_parallelize(training=True)``); every tensor rank
              sees the same rows of the batch.
``expert``    the experts of every sparse layer are split (``parallel.ep.ExpertParallel.shard``); the axis is also a batch
              axis, so different expert ranks see different rows.
``fsdp``      optimizer state is sharded over it (``FSDPEngine``), together with ``data`` and ``expert`` unless the spec asks
              for ``replicas``.
``data`` + ``replicas``  hybrid sharding: state is sharded over ``fsdp`` (x ``expert``) only and the ``data`` axis holds whole
              replicas of that group, whose gradients are summed by an all-reduce per unit before the sharded update.
``stage``     the layer stack is cut into consecutive stages (``parallel.pp.PipelineEngine``: GPipe, activations by
              overlapped NCCL point-to-point transfers, each stage owning the optimizer state of its own layers).
``diloco``    outer replicas that average their parameter change every N steps (``Trainer(diloco=...)``).
``sequence``  activations are split along the sequence inside the layers (``parallel.sp``); it does not change the engine.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .mesh import Mesh, MeshSpec


def build_engine(trainer):
    """The engine for ``trainer.mesh`` (a ``MeshSpec``, a built ``Mesh`` or None)."""
    from ..training.trainer import LocalEngine
    spec = trainer.mesh
    if getattr(trainer, "offload", None) == "optimizer":
        if spec is not None and dist.is_initialized() and dist.get_world_size() > 1:
            raise ValueError("optimizer-state offload is a one-device engine; shard over GPUs with the fsdp axis instead")
        from ..training.offload import HostOffloadEngine
        return HostOffloadEngine(trainer)
    if spec is None:
        return LocalEngine(trainer)
    mesh: Mesh = spec.build() if isinstance(spec, MeshSpec) else spec
    if not dist.is_initialized() or mesh.world == 1:
        cfg = trainer.optimizer.config
        on_gpu = torch.cuda.is_available() and all(p.is_meta or p.is_cuda for p in trainer.objective.model.parameters())
        if (on_gpu and trainer.param_dtype == torch.bfloat16 and cfg.optimizer in ("adamw", "adam") and not cfg.param_groups
                and cfg.state_dtype == "float32"):
            # one GPU under a mesh: the sharded engine with a world of one, so 1-GPU and N-GPU runs share one code path
            return _engine_class(trainer, 1)(trainer, mesh=mesh)
        return LocalEngine(trainer)
    sizes = mesh.sizes
    model = trainer.objective.model
    replicas = getattr(mesh.spec, "replicas", 1)

    if sizes["stage"] > 1:
        from .pp import PipelineEngine
        return PipelineEngine(trainer, mesh)

    if sizes["tensor"] > 1 or sizes["expert"] > 1:
        # the model is split in place: it must hold real, initialised weights first (the same on every rank)
        if any(p.is_meta for p in model.parameters()):
            raise ValueError("tensor / expert parallelism splits real weights: build the model on a device, not on 'meta'")
        if not any(getattr(p, "expert_parallel", False) or getattr(p, "tensor_parallel", False) for p in model.parameters()):
            from ..nn.layers import reset_all
            from ..utils import keys as K
            reset_all(model, int(K.fold_in(trainer.key, "init")) & 0x7FFFFFFF)

    tensor_group = None
    if sizes["tensor"] > 1:
        from .tp import TensorParallel, tensor_parallelize
        tensor_group = mesh.group("tensor")
        dev = next((p.device for p in model.parameters() if not p.is_meta), torch.device("cpu"))
        tp = TensorParallel(tensor_group, device=dev)
        tp.fused = False                      # training runs the differentiable collectives; the fused kernel serves decoding
        tensor_parallelize(model, tp, training=True)

    if sizes["expert"] > 1:
        from .ep import ExpertParallel
        if not any(getattr(p, "expert_parallel", False) for p in model.parameters()):
            ExpertParallel(group=mesh.group("expert"), fused=next(model.parameters()).is_cuda).shard(model)

    # which axes shard the state, which replicate it
    if replicas > 1:
        shard_axes = tuple(a for a in ("expert", "fsdp") if sizes[a] > 1)
        replica_axes = ("data",) if sizes["data"] > 1 else ()
    else:
        shard_axes = tuple(a for a in ("data", "expert", "fsdp") if sizes[a] > 1)
        replica_axes = ()
    batch_axes = tuple(a for a in ("data", "expert", "fsdp") if sizes[a] > 1)
    batch_ranks = mesh.size(*batch_axes) if batch_axes else 1
    if not shard_axes and not replica_axes and tensor_group is None and sizes["expert"] == 1:
        return LocalEngine(trainer)

    cfg = trainer.optimizer.config
    fused_ok = cfg.optimizer in ("adamw", "adam") and not cfg.param_groups and cfg.state_dtype == "float32"
    if not fused_ok:
        # any other optimizer keeps whole state on every rank and sums gradients over the batch ranks (plain data parallelism)
        if tensor_group is not None or sizes["expert"] > 1:
            raise NotImplementedError(f"optimizer={cfg.optimizer!r} with tensor or expert parallelism: the sharded engine "
                                      "implements adam / adamw; use one of them on this mesh")
        return DataParallelEngine(trainer, mesh.group(*batch_axes), mesh=mesh)

    engine_cls = _engine_class(trainer, mesh.size(*shard_axes) if shard_axes else 1)
    group = mesh.group(*shard_axes) if shard_axes else None
    # rank-local (expert) parameters are complete for the rows of their expert group; ranks that hold the same experts on
    # other data / fsdp coordinates saw other rows
    local_axes = tuple(a for a in ("data", "fsdp") if sizes[a] > 1) if sizes["expert"] > 1 else ()
    engine = engine_cls(trainer, group=group if shard_axes else _self_group(),
                        replica_group=mesh.group(*replica_axes) if replica_axes else None,
                        local_group=mesh.group(*local_axes) if local_axes else None,
                        batch_ranks=batch_ranks, batch_index=mesh.index(*batch_axes) if batch_axes else 0, mesh=mesh)
    engine.tensor_group = tensor_group
    return engine


def _engine_class(trainer, shard_ranks: int):
    """``FSDPEngine`` (resident compute copy and gradient accumulators) or ``ShardedFSDPEngine`` (everything sharded), as the
    trainer's ``Layout.memory`` asks; "auto" keeps the resident layout while its unsharded state (2 + 4 bytes per parameter)
    fits in ``Layout.memory_fraction`` of the device's memory."""
    import os
    from .fsdp import FSDPEngine
    from .fsdp_sharded import ShardedFSDPEngine
    layout = trainer.layout
    mode = os.environ.get("DEWB_FSDP_MEMORY") or (getattr(layout, "memory", "auto") if layout is not None else "auto")
    if mode not in ("auto", "resident", "sharded"):
        raise ValueError(f"Layout.memory must be 'auto', 'resident' or 'sharded', got {mode!r}")
    if mode == "auto":
        n = sum(p.numel() for p in trainer.objective.model.parameters())
        unsharded = n * 6 + n * 12 / max(1, shard_ranks)
        budget = 180e9
        if torch.cuda.is_available():
            budget = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
        fraction = getattr(layout, "memory_fraction", 0.45) if layout is not None else 0.45
        mode = "resident" if (unsharded <= fraction * budget or shard_ranks == 1) else "sharded"
    return ShardedFSDPEngine if mode == "sharded" else FSDPEngine


_SELF = None


def _self_group():
    """A process group of this rank alone (an engine whose state is not sharded still runs the same code with no peers)."""
    global _SELF
    if _SELF is None:
        mine = None
        for r in range(dist.get_world_size()):
            g = dist.new_group([r])
            if r == dist.get_rank():
                mine = g
        _SELF = mine
    return _SELF


class DataParallelEngine:
    """Whole state on every rank; each step's gradients are summed over the batch ranks with one all-reduce per parameter
    (bucketed by the backend) before the configured optimizer runs.  This is the path of optimizers the sharded update kernel
    does not implement (Muon, NorMuon, Lion, LAMB, LaProp, SGD, M3).  Reference: plain data parallelism, the ``data`` axis of
    src/dew/distributed/placement.py:54-109."""

    def __init__(self, trainer, group, mesh=None):
        from ..training.trainer import LocalEngine
        self.inner = LocalEngine(trainer)
        self.group, self.mesh = group, mesh
        self.world = dist.get_world_size(group)
        self.batch_ranks, self.batch_index = self.world, dist.get_rank(group)
        self.t = trainer
        self.inner.grad_sync = self._sync

    def _sync(self, params, mass):
        """Sum gradients and the pooled mass over the ranks (called by the local engine between backward and update)."""
        for p in params:
            if p.grad is not None:
                dist.all_reduce(p.grad, group=self.group)
        m = torch.as_tensor(float(mass), dtype=torch.float64, device=next(iter(params)).device).reshape(1)
        dist.all_reduce(m, group=self.group)
        return float(m)

    def fresh_state(self, key):
        return self.inner.fresh_state(key)

    def adopt(self, state):
        return self.inner.adopt(state)

    def step(self, state, batch):
        return self.inner.step(state, batch)

    @property
    def compute(self):
        return self.inner.compute
