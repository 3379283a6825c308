"""FSDP engine: optimizer state (fp32 masters, Adam moments, EMA) sharded over the ``fsdp`` (and ``data``) axis, with a
resident gathered compute copy of the parameters and a full fp32 gradient accumulator on every rank.

In ZeRO terms this is stage 1-2 for memory (masters / moments / EMA are sharded, the bf16 parameters and the fp32
gradient accumulators are not) with stage-3 placement of the update.  Design for one NVSwitch box with 180 GB per GPU:

* A **unit** is the embedding, one decoder layer, or the final norm + head.  Each unit's parameters live in one flat
  bf16 buffer; each rank owns one contiguous *leading* shard of it (the reference's measured choice of leading-dim
  shards, src/dew/mesh.py:84-93) as fp32 master + Adam moments.
* Per step, per unit, ONE kernel (``dewb_rs_adamw_ag``) does the gradient reduce-scatter (P2P pulls from the peers'
  fp32 gradient buffers), the AdamW update of the shard and the parameter all-gather (P2P pushes of the new bf16
  weights into every rank's full buffer).  It runs on a side stream as soon as the unit's backward has finished,
  overlapping the backward of earlier layers.  Cross-rank ordering is two sequence-numbered flags per unit in
  symmetric memory, every wait bounded.
* The gathered bf16 copy stays resident for the whole step (16 GB for an 8 B model), so microbatches never re-gather;
  with gradient clipping the kernel runs in two phases around a global-norm reduction.
* ``world == 1`` is the same code with no peers, so 1-GPU and N-GPU runs share one path.

Reference behaviour covered: sharded placement of masters, optimizer state and EMA
(src/dew/distributed/placement.py:54-109), microbatch accumulation, skip_nonfinite, clip_grads, EMA
(src/dew/training/transaction.py:1292-1392).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..objectives.base import Aux, Step, pool
from ..ops import library as L
from ..training.state import TrainState
from ..utils import keys as K
from ..utils.trees import flatten, module_path_to_tree_path, unflatten
from .symm import SymmetricBuffer

ALIGN = 64          # elements; keeps every parameter 128-byte aligned inside the flat buffer (TMA needs 16 bytes)
SLOT_READY, SLOT_DONE = 0, 1


def default_units(model: nn.Module) -> List[Tuple[str, List[nn.Module]]]:
    """Embedding | each layer | everything else (final norm, head), in forward order."""
    layers = getattr(model, "layers", None) or getattr(model, "blocks", None)
    if layers is None:
        return [("model", [model])]
    inside = set()
    for l in layers:
        inside.update(id(p) for p in l.parameters())
    pre, post = [], []
    seen_layers = False
    for name, child in model.named_children():
        if child is layers:
            seen_layers = True
            continue
        (post if seen_layers else pre).append(child)
    units = []
    if pre:
        units.append(("pre", pre))
    units += [(f"layer{i}", [l]) for i, l in enumerate(layers)]
    if post:
        units.append(("post", post))
    return units


@dataclass
class Unit:
    name: str
    params: List[Tuple[str, nn.Parameter]]
    offset: int = 0            # element offset of the unit inside the arenas
    size: int = 0              # padded size (multiple of world * ALIGN)
    decay_end: int = 0         # elements [0, decay_end) take weight decay
    offsets: Dict[str, int] = field(default_factory=dict)
    world: int = 1             # ranks the unit is sharded over: the engine's group, or 1 for rank-local (expert-parallel) units
    rank: int = 0
    shard_offset: int = 0      # element offset of this rank's shard inside master / moments / EMA
    group: int = 0             # index of the module group (one backward boundary) the unit belongs to

    @property
    def shard_size(self) -> int:
        return self.size // self.world

    @property
    def local(self) -> bool:
        return self.world == 1


class _Boundary(torch.autograd.Function):
    """Identity on the unit's input whose backward marks "every gradient of this unit has been produced"."""

    @staticmethod
    def forward(ctx, x, engine, index):
        ctx.engine, ctx.index = engine, index
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.engine._unit_backward_done(ctx.index)
        return g, None, None


class FSDPEngine:
    def __init__(self, trainer, units: Optional[List[Tuple[str, List[nn.Module]]]] = None, group=None,
                 wait_limit_s: float = 20.0, comm_blocks: int = 148, replica_group=None, local_group=None,
                 batch_ranks: Optional[int] = None, batch_index: Optional[int] = None, mesh=None):
        """``group``: the ranks the state is sharded over.  ``replica_group`` (hybrid sharding): ranks that hold the same
        shard on another replica of the sharded group; each unit's gradients are summed over it before the sharded update.
        ``local_group``: the ranks over which rank-local (expert-parallel) units' gradients are summed - those that hold the
        same experts and saw other rows.  ``batch_ranks`` / ``batch_index``: how many ranks see different rows of the global
        batch, and this rank's index among them (defaults: the sharded group times the replicas)."""
        self.t = trainer
        self.model: nn.Module = trainer.objective.model
        self.group = group
        self.mesh = mesh
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.replica_group, self.local_group = replica_group, local_group
        self.replicas = dist.get_world_size(replica_group) if (replica_group is not None and dist.is_initialized()) else 1
        self.batch_ranks = batch_ranks if batch_ranks is not None else self.world * self.replicas
        self.batch_index = batch_index if batch_index is not None else self.rank
        self.wait_limit_ns = int(wait_limit_s * 1e9)
        self.comm_blocks = comm_blocks
        self.unit_modules = units or default_units(self.model)
        self.units: List[Unit] = []
        self.seq = 0
        self.built = False
        self._pending: List[int] = []
        self._last_micro = False
        self._hooks: List[Any] = []
        dev = next(self.model.parameters()).device
        if dev.type == "meta":
            dev = torch.device(getattr(trainer, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu"))
            if dev.type == "cuda" and dev.index is None:
                dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        self.cuda = self.device.type == "cuda"

    # ------------------------------------------------------------------ construction
    def _is_spared(self, name: str, p: nn.Parameter) -> bool:
        kind = getattr(p, "dew_kind", "")
        return kind in ("scale", "bias", "embedding", "sinks") or p.dim() < 2

    def build(self) -> None:
        if self.built:
            return
        cfg = self.t.optimizer.config
        # the fused kernel implements AdamW (decay on matrices, none on scales / biases / embeddings) with fp32 state; a run
        # configured otherwise would silently train with a different rule, so it is refused here
        refused = []
        if cfg.optimizer not in ("adamw", "adam"):
            refused.append(f"optimizer={cfg.optimizer!r} (the sharded update kernel implements adam / adamw)")
        if cfg.param_groups:
            refused.append("param_groups (per-group learning-rate scales / weight decay)")
        if cfg.state_dtype != "float32":
            refused.append(f"state_dtype={cfg.state_dtype!r} (moments are fp32)")
        if tuple(cfg.spared) != tuple(type(cfg)().spared):
            refused.append("a custom `spared` list (the kernel spares scales, biases, embeddings and sinks)")
        if refused:
            raise NotImplementedError("FSDPEngine does not support: " + "; ".join(refused) +
                                      ". Use adamw with the default groups, or a mesh without fsdp / data sharding.")
        self._adam_decay = cfg.weight_decay if cfg.optimizer == "adamw" else 0.0
        W = self.world
        seen = set()
        total = 0
        shard_total = 0
        self.groups: List[List[int]] = []
        covered = {id(p) for _, mods in self.unit_modules for m in mods for p in m.parameters()}
        # parameters held by the model itself rather than by one of the unit modules (a vocabulary-parallel head) join the last unit
        leftovers = [(n, p) for n, p in self.model.named_parameters() if id(p) not in covered]
        for gi, (uname, mods) in enumerate(self.unit_modules):
            named: List[Tuple[str, nn.Parameter]] = []
            for m in mods:
                prefix = next((n for n, mm in self.model.named_modules() if mm is m), "")
                for n, p in m.named_parameters():
                    if id(p) in seen:
                        continue
                    seen.add(id(p))
                    named.append(((prefix + "." + n) if prefix else n, p))
            if gi == len(self.unit_modules) - 1:
                named += leftovers
            # parameters that are already one rank's slice of an expert-parallel layer form a rank-local unit: their
            # gradients are complete on this rank (every token routed here contributed), so nothing is reduced or gathered
            shared = [(n, p) for n, p in named if not getattr(p, "expert_parallel", False)]
            local = [(n, p) for n, p in named if getattr(p, "expert_parallel", False)]
            members = []
            for suffix, plist, uw, ur in (("", shared, W, self.rank), (".local", local, 1, 0)):
                if not plist:
                    continue
                decay = [(n, p) for n, p in plist if not self._is_spared(n, p)]
                spared = [(n, p) for n, p in plist if self._is_spared(n, p)]
                u = Unit(uname + suffix, decay + spared, world=uw, rank=ur, group=gi)
                off = 0
                for i, (n, p) in enumerate(u.params):
                    if i == len(decay):
                        u.decay_end = off
                    u.offsets[n] = off
                    off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
                if not spared:
                    u.decay_end = off
                quantum = uw * ALIGN
                u.size = (off + quantum - 1) // quantum * quantum
                u.offset = total
                u.shard_offset = shard_total
                total += u.size
                shard_total += u.shard_size
                members.append(len(self.units))
                self.units.append(u)
            self.groups.append(members)
        self.total = total
        self.shard_total = shard_total
        self.compute_dtype = self.t.param_dtype or (torch.bfloat16 if self.cuda else torch.float32)
        self._allocate()
        self.device = self.params_arena.tensor.device if getattr(self, "params_arena", None) is not None else self.device
        self.built = True

    def _allocate(self) -> None:
        """Device memory of the resident layout: the full compute-dtype parameters and the full fp32 gradient accumulators
        (both peer-visible), this rank's fp32 masters and moments, and the parameters re-pointed into the arenas."""
        total, shard_total, W = self.total, self.shard_total, self.world
        dev = self.device
        cdtype = self.compute_dtype
        # arenas: full compute-dtype parameters and full fp32 gradients (peer-visible), flags
        self.params_arena = SymmetricBuffer(total, cdtype, dev, self.group, zero=True)
        self.grads_arena = SymmetricBuffer(total, torch.float32, dev, self.group, zero=True)
        self.flags = SymmetricBuffer(max(64, len(self.units) * 2 * max(W, 1)), torch.int32, dev, self.group, zero=True)
        # kernels of rank-local units run with a world of one and index their flags as `slot`, not `slot * W + rank`: they
        # get an array of their own so that they cannot touch the flags the sharded units' hand-shakes wait on
        self.local_flags = torch.zeros(max(64, len(self.units) * 2), dtype=torch.int32, device=dev)
        self.master = torch.empty(shard_total, dtype=torch.float32, device=dev)
        self.m = torch.zeros(shard_total, dtype=torch.float32, device=dev)
        self.v = torch.zeros(shard_total, dtype=torch.float32, device=dev)
        self.ema = None
        self.block_counter = torch.zeros(len(self.units), dtype=torch.int32, device=dev)
        self.clip = torch.zeros(4, dtype=torch.float32, device=dev)
        self.norm_parts = SymmetricBuffer(64, torch.float32, dev, self.group, zero=True) if W > 1 else None
        # move parameters into the arena (one at a time, releasing the original storage)
        pa, ga = self.params_arena.tensor, self.grads_arena.tensor
        self.was_meta = any(p.is_meta for u in self.units for _, p in u.params)
        owners = {}
        for mod in self.model.modules():
            for pname, p in mod._parameters.items():
                if p is not None:
                    owners.setdefault(id(p), []).append((mod, pname))
        with torch.no_grad():
            for u in self.units:
                fresh = []
                for n, p in u.params:
                    o = u.offset + u.offsets[n]
                    view = pa[o:o + p.numel()].view(p.shape)
                    if p.is_meta:
                        # a model built on the meta device is materialised straight inside the arena
                        new = nn.Parameter(torch.empty(0, dtype=view.dtype, device=view.device), requires_grad=p.requires_grad)
                        new.data = view     # .data assignment gives the parameter its own version counter
                        for attr in ("logical_axes", "dew_kind"):
                            if hasattr(p, attr):
                                setattr(new, attr, getattr(p, attr))
                        for mod, pname in owners[id(p)]:
                            mod._parameters[pname] = new
                        p = new
                    else:
                        view.copy_(p.data)
                        p.data = view
                    p.main_grad = ga[o:o + p.numel()].view(p.shape)
                    p.grad = None
                    fresh.append((n, p))
                u.params = fresh

    def init_masters(self) -> None:
        """fp32 masters (and EMA) from the compute-dtype arena: this rank's shard of every unit."""
        W = self.world
        pa = self.params_arena.tensor
        with torch.no_grad():
            for u in self.units:
                s = u.shard_size
                src = pa[u.offset + u.rank * s: u.offset + (u.rank + 1) * s]
                self.master[u.shard_offset: u.shard_offset + s].copy_(src)
        if self.t.objective.ema_spec() is not None:
            self.ema = self.master.clone()
    def _install_hooks(self) -> None:
        dev = self.device
        # unit boundaries: a backward marker at each unit's input
        for i, (uname, mods) in enumerate(self.unit_modules):
            first = mods[0]
            self._hooks.append(first.register_forward_pre_hook(self._make_pre_hook(i), with_kwargs=True))
        self.comm_stream = torch.cuda.Stream(device=dev) if self.cuda else None
        self.scratch = torch.empty(2048, dtype=torch.float32, device=dev)
        self.reduced = None

    def _make_pre_hook(self, index: int):
        def hook(module, args, kwargs):
            self._before_unit_forward(index)
            if not torch.is_grad_enabled():
                return None
            new_args = list(args)
            for j, a in enumerate(new_args):
                if isinstance(a, torch.Tensor) and a.requires_grad and a.dtype.is_floating_point:
                    new_args[j] = _Boundary.apply(a, self, index)
                    return tuple(new_args), kwargs
            # the first unit's inputs (token ids) carry no gradient: it is finalised after backward returns
            return None
        return hook

    # ------------------------------------------------------------------ state
    def fresh_state(self, key: int) -> TrainState:
        from ..nn.layers import reset_all
        if not self.built:
            seed = int(K.fold_in(key, "init")) & 0x7FFFFFFF                   # same seed on every rank
            meta = any(p.is_meta for p in self.model.parameters())
            # a model whose experts were already split over the ranks was initialised (same seed) before the split
            presharded = any(getattr(p, "expert_parallel", False) or getattr(p, "tensor_parallel", False) for p in self.model.parameters())
            if not meta and not presharded:
                reset_all(self.model, seed)
            self.build()
            if meta:
                reset_all(self.model, seed)
            self.init_masters()
            self._install_hooks()
        state = TrainState(key=key)
        state.variables = {"params": self._shard_tree(self.master)}
        state.opt_state = {"count": torch.zeros((), dtype=torch.int64), "mu": self._shard_tree(self.m), "nu": self._shard_tree(self.v)}
        state.ema = {"params": self._shard_tree(self.ema)} if self.ema is not None else None
        return state

    def _shard_tree(self, flat: torch.Tensor) -> Dict[str, Any]:
        """Expose a sharded flat buffer as a tree: one leaf per unit (``<unit>/shard``) holding this rank's shard."""
        return unflatten({f"{u.name}/shard": flat[u.shard_offset: u.shard_offset + u.shard_size] for u in self.units})

    def adopt(self, state: TrainState) -> TrainState:
        if not self.built:
            self.build()
            self.init_masters()
            self._install_hooks()
        return state

    def _whole_unit(self, u: Unit, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        """The unit's tensors in full, by parameter tree path (collective over the engine's group).  A sharded unit is
        all-gathered; a rank-local (expert-parallel) unit holds a different slice of the experts on every rank, so the
        ranks' copies are concatenated along the expert dimension."""
        W = self.world
        mine = flat[u.shard_offset: u.shard_offset + u.shard_size]
        out: Dict[str, torch.Tensor] = {}
        if W == 1:
            for n, p in u.params:
                o = u.offsets[n]
                out[module_path_to_tree_path(n)] = mine[o:o + p.numel()].view(p.shape)
            return out
        if u.local:
            every = torch.empty(W * u.size, dtype=flat.dtype, device=flat.device)
            dist.all_gather_into_tensor(every, mine.contiguous(), group=self.group)
            every = every.view(W, u.size)
            for n, p in u.params:
                o = u.offsets[n]
                out[module_path_to_tree_path(n)] = every[:, o:o + p.numel()].reshape((W * p.shape[0],) + tuple(p.shape[1:]))
            return out
        full = torch.empty(u.size, dtype=flat.dtype, device=flat.device)
        dist.all_gather_into_tensor(full, mine.contiguous(), group=self.group)
        for n, p in u.params:
            o = u.offsets[n]
            out[module_path_to_tree_path(n)] = full[o:o + p.numel()].view(p.shape)
        return out

    def gather_full(self, what: str = "master") -> Dict[str, torch.Tensor]:
        """Full (unsharded) fp32 tensors by parameter tree path - for checkpoints and evaluation on rank 0."""
        flat = {"master": self.master, "mu": self.m, "nu": self.v, "ema": self.ema}[what]
        out: Dict[str, torch.Tensor] = {}
        for u in self.units:
            for k, v in self._whole_unit(u, flat).items():
                out[k] = v.clone()
        return out

    # ------------------------------------------------------------------ checkpoints (layout-free full trees)
    def export_state(self, state: TrainState, to: str = "cpu") -> Optional[TrainState]:
        """Collective.  The state with whole (unsharded) fp32 trees keyed by parameter path, as a checkpoint stores it,
        so a checkpoint written at one world size restores at another.  Units are gathered one at a time and moved to
        ``to`` on rank 0 only; other ranks return None."""
        keep = self.rank == 0

        def whole(flat):
            if flat is None:
                return None
            out: Dict[str, torch.Tensor] = {}
            for u in self.units:
                for k, v in self._whole_unit(u, flat).items():
                    if keep:
                        out[k] = v.to(to, copy=True)
            return unflatten(out)

        trees = {k: whole(v) for k, v in (("params", self.master), ("mu", self.m), ("nu", self.v), ("ema", self.ema))}
        if not keep:
            return None
        import dataclasses as _dc
        full = _dc.replace(state)
        full.variables = {"params": trees["params"]}
        full.opt_state = {"count": state.opt_state["count"].to(to) if isinstance(state.opt_state.get("count"), torch.Tensor) else state.opt_state.get("count"),
                          "mu": trees["mu"], "nu": trees["nu"]}
        full.ema = {"params": trees["ema"]} if trees["ema"] is not None else None
        return full

    def import_state(self, full: TrainState, state: TrainState) -> TrainState:
        """Every rank reads a whole-tree state (e.g. a restored checkpoint) and copies the slices that fall into its own
        shards; the compute-dtype arena is then rebuilt from the new masters.  Returns ``state`` with counters adopted."""
        W, r = self.world, self.rank

        def scatter(tree, flat):
            if tree is None or flat is None:
                return
            leaves = flatten(tree)
            with torch.no_grad():
                for u in self.units:
                    s = u.shard_size
                    lo, hi = u.rank * s, (u.rank + 1) * s                         # this rank's range inside the unit
                    base = u.shard_offset
                    for n, p in u.params:
                        src = leaves.get(module_path_to_tree_path(n))
                        if src is None:
                            raise KeyError(f"checkpoint lacks {module_path_to_tree_path(n)}")
                        if u.local and W > 1:
                            # the checkpoint holds every rank's experts along the leading dimension: keep this rank's
                            src = src[r * p.shape[0]:(r + 1) * p.shape[0]]
                        o = u.offsets[n]
                        a, b = max(o, lo), min(o + p.numel(), hi)
                        if a < b:
                            flat[base + a - lo: base + b - lo].copy_(src.reshape(-1)[a - o: b - o])

        scatter(full.variables["params"], self.master)
        scatter(full.opt_state.get("mu"), self.m)
        scatter(full.opt_state.get("nu"), self.v)
        if self.ema is not None:
            scatter((full.ema or full.variables)["params"], self.ema)
        self.refresh_compute_copy()
        for f in ("step", "microstep", "updates", "consumed", "key", "deferred"):
            if hasattr(full, f):
                setattr(state, f, getattr(full, f))
        c = full.opt_state.get("count")
        if c is not None:
            state.opt_state["count"] = torch.as_tensor(c).to(torch.int64)
        return state

    def refresh_compute_copy(self) -> None:
        """Rebuild every rank's full compute-dtype parameters from the fp32 master shards (an all-gather)."""
        W = self.world
        pa = self.params_arena.tensor
        with torch.no_grad():
            for u in self.units:
                mine = self.master[u.shard_offset: u.shard_offset + u.shard_size].to(pa.dtype)
                if W > 1 and not u.local:
                    dist.all_gather_into_tensor(pa[u.offset: u.offset + u.size], mine, group=self.group)
                else:
                    pa[u.offset: u.offset + u.size].copy_(mine)
        if self.cuda:
            torch.cuda.synchronize(self.device)
        if W > 1:
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ per-unit protocol
    def _before_unit_forward(self, group: int) -> None:
        """First forward of a module group in a step: wait until every peer's push of its new weights has landed and
        the peers have stopped reading its gradient buffer, then clear that buffer."""
        if not self._first_micro or group in self._cleared:
            return
        self._cleared.add(group)
        for index in self.groups[group]:
            u = self.units[index]
            if self.cuda and self.world > 1 and self.seq > 0 and not u.local and getattr(self, "_synced_seq", -1) != self.seq:
                L.check(L.load().dewb_wait_flags(L.ptr(self.flags.tensor), ctypes.c_int(index * 2 + SLOT_DONE),
                                                 ctypes.c_int(self.world), ctypes.c_uint(self.seq),
                                                 ctypes.c_ulonglong(self.wait_limit_ns), L.ptr(L.status(self.device)),
                                                 L.stream_ptr()), "wait_flags")
                L.count_launches()
            self.grads_arena.tensor[u.offset:u.offset + u.size].zero_()

    def _await_pushes(self) -> None:
        """After a step: this rank's stream waits (bounded) until every peer's push of every unit's new weights has landed
        in this rank's parameter arena, so whatever runs next on it - an evaluation, a preview, a checkpoint export, the
        next step's first forward - reads whole weights of the new step.  One tiny kernel per sharded unit."""
        if not (self.cuda and self.world > 1 and self.seq > 0):
            return
        lib = L.load()
        for index, u in enumerate(self.units):
            if u.local:
                continue
            L.check(lib.dewb_wait_flags(L.ptr(self.flags.tensor), ctypes.c_int(index * 2 + SLOT_DONE), ctypes.c_int(self.world),
                                        ctypes.c_uint(self.seq), ctypes.c_ulonglong(self.wait_limit_ns),
                                        L.ptr(L.status(self.device)), L.stream_ptr()), "wait_flags")
            L.count_launches()
        self._synced_seq = self.seq

    def _unit_backward_done(self, group: int) -> None:
        if not self._last_micro or group in self._launched:
            return
        self._finalize_unit(group)

    def _fold_autograd_grads(self, u: Unit) -> None:
        """Gradients that arrived through autograd's ``.grad`` (norm scales, embeddings) join the fp32 accumulators."""
        for n, p in u.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None

    def _sum_over(self, u: Unit, group) -> None:
        """Sum the unit's fp32 gradient accumulator over ``group`` (NCCL / gloo all-reduce, on the communication stream on a
        GPU so it overlaps the backward of earlier layers)."""
        g = self.grads_arena.tensor[u.offset:u.offset + u.size]
        if self.cuda:
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.comm_stream):
                dist.all_reduce(g, group=group)
        else:
            dist.all_reduce(g, group=group)

    def _finalize_unit(self, group: int) -> None:
        self._launched.add(group)
        for index in self.groups[group]:
            u = self.units[index]
            self._fold_autograd_grads(u)
            if u.local and self.local_group is not None:
                self._sum_over(u, self.local_group)
            elif not u.local and self.replica_group is not None:
                self._sum_over(u, self.replica_group)
            self._launch(index, mode=1 if self._two_phase else 0)

    def _hyper(self, u: Unit):
        cfg = self.t.optimizer.config
        o = cfg.optimizer_opts
        b1, b2 = o.get("b1", 0.9), o.get("b2", 0.999)
        count = self._count
        ema_decay = 0.0
        spec = self.t.objective.ema_spec()
        if spec is not None:
            ema_decay = spec.at(self._updates + 1)
        vals = [self._lr, b1, b2, o.get("eps", 1e-8), self._adam_decay, 1 - b1 ** count, 1 - b2 ** count,
                self._grad_scale, ema_decay]
        return (ctypes.c_float * 9)(*vals)

    def _launch(self, index: int, mode: int) -> None:
        u = self.units[index]
        W, r = u.world, u.rank
        s = u.shard_size
        lo = u.shard_offset
        if not self.cuda:
            return self._launch_reference(u, mode)
        lib = L.load()
        cur = torch.cuda.current_stream(self.device)
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            esz = self.params_arena.tensor.element_size()
            own = u.local and self.world > 1          # a rank-local unit sees only this rank's buffers
            rc = lib.dewb_rs_adamw_ag(
                self.grads_arena.own_ptr_array(u.offset * 4) if own else self.grads_arena.ptr_array(u.offset * 4),
                self.params_arena.own_ptr_array(u.offset * esz) if own else self.params_arena.ptr_array(u.offset * esz),
                (ctypes.c_ulonglong * 8)(*([self.local_flags.data_ptr()] + [0] * 7)) if own else self.flags.ptr_array(),
                L.ptr(self.master[lo:lo + s]), L.ptr(self.m[lo:lo + s]), L.ptr(self.v[lo:lo + s]),
                L.ptr(self.ema[lo:lo + s] if self.ema is not None else None),
                L.ptr(self.reduced[lo:lo + s] if self.reduced is not None else None),
                L.ptr(self.sumsq[index] if self._two_phase else None),
                L.ptr(self.clip if mode == 2 else None),
                ctypes.c_longlong(r * s), ctypes.c_longlong(s), ctypes.c_longlong(u.decay_end), ctypes.c_int(r),
                ctypes.c_int(W), self._hyper(u), ctypes.c_uint(self.seq + 1), ctypes.c_int(index * 2 + SLOT_READY),
                ctypes.c_int(index * 2 + SLOT_DONE), L.ptr(self.block_counter[index:index + 1]),
                ctypes.c_ulonglong(self.wait_limit_ns), ctypes.c_int(mode),
                ctypes.c_int(int(self.t.optimizer.config.skip_nonfinite)), ctypes.c_int(self.comm_blocks),
                L.ptr(L.status(self.device)), ctypes.c_void_p(self.comm_stream.cuda_stream))
            L.check(rc, "rs_adamw_ag")
            L.count_launches()

    def _launch_reference(self, u: Unit, mode: int) -> None:
        """CPU path (gloo ranks): the same arithmetic with torch collectives - the oracle for the fused kernel."""
        W, r = u.world, u.rank
        s = u.shard_size
        lo = u.shard_offset
        g_full = self.grads_arena.tensor[u.offset:u.offset + u.size]
        if W > 1:
            g = torch.empty(s, dtype=torch.float32)
            dist.reduce_scatter_tensor(g, g_full.contiguous(), group=self.group)
        else:
            g = g_full.clone()
        if mode == 1:
            self.reduced[lo:lo + s].copy_(g)
            self.sumsq[self.units.index(u)].zero_()
            self.sumsq[self.units.index(u)][0] = g.pow(2).sum()
            return
        if mode == 2:
            g = self.reduced[lo:lo + s]
        h = list(self._hyper(u))
        lr, b1, b2, eps, wd, bc1, bc2, gs, ed = h
        coef = gs * (float(self.clip[2]) if mode == 2 else 1.0)
        if mode == 2 and self.t.optimizer.config.skip_nonfinite and not math.isfinite(float(self.clip[0])):
            return
        g = g * coef
        m, v, p = self.m[lo:lo + s], self.v[lo:lo + s], self.master[lo:lo + s]
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        idx = torch.arange(r * s, (r + 1) * s)
        wdv = torch.where(idx < u.decay_end, torch.tensor(wd), torch.tensor(0.0))
        p.mul_(1 - lr * wdv).addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
        if self.ema is not None:
            self.ema[lo:lo + s].mul_(ed).add_(p, alpha=1 - ed)
        full = self.params_arena.tensor[u.offset:u.offset + u.size]
        if W > 1:
            dist.all_gather_into_tensor(full, p.to(full.dtype).contiguous(), group=self.group)
        else:
            full.copy_(p)

    # ------------------------------------------------------------------ the step
    def step(self, state: TrainState, batch: Mapping[str, torch.Tensor]):
        from ..ops import mx as _mx
        _mx.cache_weights(True) if not _mx._CACHE_ON[0] else None
        _mx.weights_changed()          # whatever changed the weights since the last step (a restore, a reload), quantised copies start afresh
        from ..training.trainer import _split_rows, tree_detach
        t = self.t
        obj = t.objective
        cfg = t.optimizer.config
        parts = _split_rows(batch, t.microbatches or 1)
        step_key = K.fold_in(state.key, state.step)
        self._lr = float(t.optimizer.schedule(state.step))
        self._count = int(state.opt_state["count"]) + 1
        self._updates = state.updates
        self._two_phase = cfg.clip_grads is not None or cfg.skip_nonfinite
        if self._two_phase and self.reduced is None:
            self.reduced = torch.zeros(self.shard_total, dtype=torch.float32, device=self.device)
            self.sumsq = torch.zeros(len(self.units), max(self.comm_blocks, 1), dtype=torch.float32, device=self.device)
        self._cleared, self._launched = set(), set()
        stats_all, metrics_all, effects = [], {}, {}
        mass_total = None
        rows_per = next(iter(parts[0].values())).shape[0]
        # the pooled mass scales every gradient: it is known before the backward of the last microbatch only if the
        # objective can count it from the batch (token counts); otherwise fall back to rows
        mass_known = None
        if hasattr(obj, "scored_tokens"):
            try:
                mass_known = float(sum(obj.scored_tokens(mb) or 0 for mb in parts))
            except Exception:
                mass_known = None
        if mass_known is None or mass_known <= 0:
            mass_known = float(rows_per * len(parts))
        if self.batch_ranks > 1:
            uniform = getattr(obj, "uniform_mass", None)
            if not hasattr(obj, "scored_tokens") or (callable(uniform) and all(uniform(mb) for mb in parts)):
                # every rank scores the same number of targets (no padding, equal rows): no exchange, no host sync
                mass_known = mass_known * self.batch_ranks
            else:
                mk = torch.tensor([mass_known], dtype=torch.float64, device=self.device)
                dist.all_reduce(mk, group=self.group)
                if self.replica_group is not None:
                    dist.all_reduce(mk, group=self.replica_group)
                mass_known = float(mk.item()) * self.batch_ranks / (self.world * self.replicas)
        self._grad_scale = 1.0 / max(mass_known, 1e-12)
        first = self.batch_index * rows_per * len(parts)
        for i, mb in enumerate(parts):
            self._first_micro = i == 0
            self._last_micro = i == len(parts) - 1
            st = Step(step=state.step, key=step_key, ema=None, train=True, first_index=first, device=self.device)
            out = obj.loss(None, mb, st)
            stats, aux = out if isinstance(out, tuple) else (out, Aux())
            total, mass = obj.reduce_loss(stats)
            total.backward()
            stats_all.append(tree_detach(stats))
            for k, v in aux.metrics.items():
                metrics_all.setdefault(k, []).append(tree_detach(v))
            effects.update(aux.effects)
            first += rows_per
        # units whose input carries no gradient (the embedding) are finalised here, in reverse order
        for group in reversed(range(len(self.groups))):
            if group not in self._launched:
                self._finalize_unit(group)
        info: Dict[str, Any] = {"learning_rate": self._lr}
        if self._two_phase:
            self._second_phase(info)
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        self.seq += 1
        self._await_pushes()
        # a step whose gradient norm was not finite changed nothing (the kernel left masters, moments and EMA alone): the
        # update count and the EMA schedule do not advance either
        skipped = bool(self._two_phase and cfg.skip_nonfinite and not math.isfinite(float(self.clip[0])))
        if skipped:
            info["skipped"] = True
        else:
            obj.apply_effects(state.variables, effects)
        new_opt = dict(state.opt_state)
        new_opt["count"] = torch.tensor(self._count - (1 if skipped else 0), dtype=torch.int64)
        rows_total = rows_per * len(parts) * self.batch_ranks
        new_state = state.replace(step=state.step + 1, microstep=state.microstep + len(parts),
                                  updates=state.updates + (0 if skipped else 1), opt_state=new_opt,
                                  consumed={"examples": state.consumed.get("examples", 0) + rows_total,
                                            "tokens": state.consumed.get("tokens", 0) + int(obj.row_tokens(batch) or 0) * self.batch_ranks})
        pooled = pool(stats_all)
        metrics = {"loss": pooled, **{k: pool(v) for k, v in metrics_all.items()}, **info}
        _mx.weights_changed()          # the update just written makes this step's quantised copies stale for whoever runs next
        return new_state, metrics

    def _second_phase(self, info: Dict[str, Any]) -> None:
        """Global gradient norm from the per-unit partial sums, then the AdamW + push phase for every unit."""
        cfg = self.t.optimizer.config
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        local = self.sumsq.sum().reshape(1) * (self._grad_scale ** 2)
        tensor_group = getattr(self, "tensor_group", None)
        if tensor_group is not None:
            # under tensor parallelism every tensor rank holds other slices of the sharded matrices but the SAME norm scales
            # and embeddings: those are counted once, the sharded ones summed over the tensor ranks
            rep = torch.zeros(1, dtype=torch.float32, device=self.device)
            for u in self.units:
                s_, lo_ = u.shard_size, u.rank * u.shard_size
                for n, p in u.params:
                    if getattr(p, "tensor_parallel", False):
                        continue
                    o = u.offsets[n]
                    a, b = max(o, lo_), min(o + p.numel(), lo_ + s_)
                    if a < b:
                        rep += self.reduced[u.shard_offset + a - lo_: u.shard_offset + b - lo_].pow(2).sum()
            rep = rep * (self._grad_scale ** 2)
            sharded = local - rep
            dist.all_reduce(sharded, group=tensor_group)
            local = sharded + rep
        if self.world > 1:
            dist.all_reduce(local, group=self.group)
        norm = local.sqrt()
        self.clip[0:1] = local
        self.clip[1:2] = norm
        maxn = cfg.clip_grads
        self.clip[2:3] = torch.where((norm > maxn), maxn / (norm + 1e-6), torch.ones_like(norm)) if maxn else torch.ones_like(norm)
        info["grad_norm"] = self.clip[1].clone()
        for index in reversed(range(len(self.units))):
            self._launch(index, mode=2)

    def close(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
