"""Fully sharded engine (ZeRO-3 memory model): parameters, gradients and optimizer state all live as one shard per rank.

Where ``FSDPEngine`` keeps a gathered compute copy of every parameter and a full fp32 gradient accumulator resident on
every rank (fastest while they fit), this engine keeps, per rank:

* the bf16 **shard** of every unit's parameters (peer-visible), fp32 master / moments / EMA shards and an fp32 gradient
  accumulator **of the shard only**;
* ``gather_slots`` (3) buffers of the largest unit's size, into which a unit's parameters are all-gathered just before its
  forward and again before its backward - a pull over NVLink from the peers' shards, issued on the communication stream
  one unit ahead of the compute stream;
* 2 peer-visible fp32 gradient buffers of the largest unit's size: a unit's backward writes its gradients there, and one
  kernel (``dewb_rs_adamw_ag`` in its accumulate mode) announces them, waits (bounded) for every peer's, pulls this rank's
  range from every peer, adds the sum into the shard accumulator and tells the peers their buffer may be reused.

After the last microbatch AdamW runs on the shards and each rank rewrites its own bf16 shard.  Per step a model of P
parameters on W ranks therefore holds ``P / W x (2 + 4 + 4 + 4 + 4)`` bytes of state plus five unit-sized buffers, instead of
``P x 6`` bytes of unsharded state; the price is one parameter all-gather per unit per forward and per backward and one
gradient reduce-scatter per unit per microbatch.

Reference: leading-dimension shards (src/dew/mesh.py:162-218), state that follows the shard
(src/dew/distributed/placement.py:54-109), the per-layer gather budget (src/dew/training/memory.py:69-100).
"""
from __future__ import annotations

import ctypes
import math
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import library as L
from ..training.state import TrainState
from ..utils import keys as K
from .fsdp import SLOT_DONE, SLOT_READY, FSDPEngine, Unit
from .symm import SymmetricBuffer


class ShardedFSDPEngine(FSDPEngine):
    def __init__(self, trainer, *args, gather_slots: int = 3, **kw):
        super().__init__(trainer, *args, **kw)
        if gather_slots < 3:
            raise ValueError("gather_slots must be at least 3: the unit in use, the one being prefetched and the one just left")
        self.n_gather = gather_slots
        self.rs_seq = 0                       # one sequence number per (step, microbatch): gradient hand-shakes
        self._init_seed: Optional[int] = None

    # ------------------------------------------------------------------ construction
    def _allocate(self) -> None:
        W, dev, cd = self.world, self.device, self.compute_dtype
        model = self.model
        if getattr(getattr(model, "config", None), "tie_embeddings", False) and getattr(model, "head", 1) is None \
                and getattr(model, "tp_head", None) is None:
            raise NotImplementedError("the fully sharded engine needs an untied head: a tied table is used by the first and the "
                                      "last unit, whose parameters are gathered at different times")
        # the units of one module group (its sharded parameters and, under expert parallelism, its rank-local ones) share a
        # buffer, one after the other; buffers are assigned by group index
        slot = 0
        for members in self.groups:
            at = 0
            for ui in members:
                self.units[ui].slot_base = at
                at += self.units[ui].size
            slot = max(slot, at)
        self.slot_size = slot
        self.group_of = {ui: gi for gi, members in enumerate(self.groups) for ui in members}
        self.shards = SymmetricBuffer(self.shard_total, cd, dev, self.group, zero=True)
        self.gathered = [torch.zeros(slot, dtype=cd, device=dev) for _ in range(self.n_gather)]
        self.grad_slots = [SymmetricBuffer(slot, torch.float32, dev, self.group, zero=True) for _ in range(2)]
        self.flags = SymmetricBuffer(max(64, (len(self.units) * 2 + 2) * max(W, 1)), torch.int32, dev, self.group, zero=True)
        self.sync_slot = len(self.units) * 2                       # end-of-step "my new shard is written" flags
        self.local_flags = torch.zeros(max(64, len(self.units) * 2 + 2), dtype=torch.int32, device=dev)   # kernels run with a world of one
        st = self.shard_total
        self.master = torch.empty(st, dtype=torch.float32, device=dev)
        self.m = torch.zeros(st, dtype=torch.float32, device=dev)
        self.v = torch.zeros(st, dtype=torch.float32, device=dev)
        self.reduced = torch.zeros(st, dtype=torch.float32, device=dev)          # the shard's gradient accumulator
        self.ema = None
        self.block_counter = torch.zeros(len(self.units), dtype=torch.int32, device=dev)
        self.clip = torch.zeros(4, dtype=torch.float32, device=dev)
        self.norm_parts = None
        self.params_arena = self.grads_arena = None
        self.resident: List[Optional[int]] = [None] * self.n_gather
        self.was_meta = any(p.is_meta for u in self.units for _, p in u.params)
        owners: Dict[int, list] = {}
        for mod in model.modules():
            for pname, p in mod._parameters.items():
                if p is not None:
                    owners.setdefault(id(p), []).append((mod, pname))
        seed = self._init_seed
        with torch.no_grad():
            for gi, members in enumerate(self.groups):
                for ui in members:
                    u = self.units[ui]
                    gslot = self.gathered[gi % self.n_gather][u.slot_base:u.slot_base + u.size]
                    dslot = self.grad_slots[gi % 2].tensor[u.slot_base:u.slot_base + u.size]
                    fresh, gaps, at = [], [], 0
                    for n, p in u.params:
                        o = u.offsets[n]
                        if o > at:
                            gaps.append(dslot[at:o])
                        at = o + p.numel()
                        view = gslot[o:o + p.numel()].view(p.shape)
                        if p.is_meta:
                            new = nn.Parameter(torch.empty(0, dtype=view.dtype, device=view.device), requires_grad=p.requires_grad)
                            new.data = view
                            for attr in ("logical_axes", "dew_kind", "expert_parallel", "tensor_parallel"):
                                if hasattr(p, attr):
                                    setattr(new, attr, getattr(p, attr))
                            for mod, pname in owners[id(p)]:
                                mod._parameters[pname] = new
                            p = new
                        else:
                            view.copy_(p.data)
                            p.data = view
                        p.main_grad = dslot[o:o + p.numel()].view(p.shape)
                        p.grad = None
                        fresh.append((n, p))
                    if u.size > at:
                        gaps.append(dslot[at:u.size])
                    u.params = fresh
                    u.gaps = gaps             # padding between / after the parameters: zeroed before every reduction
                if self.was_meta:
                    # a model built on the meta device is initialised unit by unit inside the gather buffers (same draws as
                    # initialising it whole), since the buffers are shared between units
                    from ..nn.layers import reset_all
                    for mod in self.unit_modules[gi][1]:
                        prefix = next((n for n, mm in model.named_modules() if mm is mod), "")
                        reset_all(mod, seed if seed is not None else 0, prefix=prefix)
                for ui in members:                   # publish this rank's shard of the unit
                    u = self.units[ui]
                    s = u.shard_size
                    gslot = self.gathered[gi % self.n_gather][u.slot_base:u.slot_base + u.size]
                    self.shards.tensor[u.shard_offset:u.shard_offset + s].copy_(gslot[u.rank * s:(u.rank + 1) * s])
        if self.cuda:
            torch.cuda.synchronize(dev)
        if W > 1:
            dist.barrier(group=self.group)

    def init_masters(self) -> None:
        with torch.no_grad():
            self.master.copy_(self.shards.tensor)
        if self.t.objective.ema_spec() is not None:
            self.ema = self.master.clone()

    def fresh_state(self, key: int) -> TrainState:
        from ..nn.layers import reset_all
        if not self.built:
            seed = int(K.fold_in(key, "init")) & 0x7FFFFFFF
            self._init_seed = seed
            meta = any(p.is_meta for p in self.model.parameters())
            presharded = any(getattr(p, "expert_parallel", False) or getattr(p, "tensor_parallel", False) for p in self.model.parameters())
            if not meta and not presharded:
                reset_all(self.model, seed)
            self.build()
            self.init_masters()
            self._install_hooks()
        state = TrainState(key=key)
        state.variables = {"params": self._shard_tree(self.master)}
        state.opt_state = {"count": torch.zeros((), dtype=torch.int64), "mu": self._shard_tree(self.m), "nu": self._shard_tree(self.v)}
        state.ema = {"params": self._shard_tree(self.ema)} if self.ema is not None else None
        return state

    def _install_hooks(self) -> None:
        accumulator = self.reduced
        super()._install_hooks()
        self.reduced = accumulator
        self.ready_events: Dict[int, Any] = {}
        self.rs_events: Dict[int, Any] = {}
        # backward of the last unit starts straight after the forward; every other unit's backward is announced by the
        # boundary of the unit after it (``_unit_backward_done``)

    def refresh_compute_copy(self) -> None:
        """Rewrite this rank's compute-dtype shard from its fp32 master shard; gathered copies are stale afterwards."""
        with torch.no_grad():
            self.shards.tensor.copy_(self.master.to(self.shards.tensor.dtype))
        self.resident = [None] * self.n_gather
        if self.cuda:
            torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ parameter gathers
    def _own_ptrs(self, tensor: torch.Tensor, offset_bytes: int = 0):
        return (ctypes.c_ulonglong * 8)(*([tensor.data_ptr() + offset_bytes] + [0] * 7))

    def _gather(self, group: int) -> None:
        """Make the parameters of ``group``'s units whole in the group's gather buffer (a pull from every peer's shard on the
        communication stream); the compute stream is made to wait for it by ``_need``."""
        slot = group % self.n_gather
        if self.resident[slot] == group:
            return
        self.resident[slot] = group
        buf = self.gathered[slot]
        if self.cuda:
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))   # all enqueued readers of the previous occupant
        for ui in self.groups[group]:
            u = self.units[ui]
            s = u.shard_size
            dst = buf[u.slot_base:u.slot_base + u.size]
            mine = self.shards.tensor[u.shard_offset:u.shard_offset + s]
            if not self.cuda:
                if u.world > 1:
                    dist.all_gather_into_tensor(dst, mine.contiguous(), group=self.group)
                else:
                    dst.copy_(mine)
                continue
            esz = dst.element_size()
            with torch.cuda.stream(self.comm_stream):
                if u.world > 1:
                    L.check(L.load().dewb_allgather_pull(self.shards.ptr_array(u.shard_offset * esz), L.ptr(dst),
                                                         ctypes.c_longlong(s * esz), ctypes.c_int(u.world),
                                                         ctypes.c_int(self.comm_blocks), ctypes.c_void_p(self.comm_stream.cuda_stream)),
                            "allgather_pull")
                    L.count_launches()
                else:
                    dst.copy_(mine, non_blocking=True)
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
            self.ready_events[group] = ev

    def _need(self, group: int) -> None:
        self._gather(group)
        if self.cuda and group in self.ready_events:
            torch.cuda.current_stream(self.device).wait_event(self.ready_events[group])

    def _group_units(self, group: int) -> List[int]:
        return self.groups[group]

    def _before_unit_forward(self, group: int) -> None:
        self._need(group)
        if group + 1 < len(self.groups):              # one group ahead, overlapping this group's compute
            self._gather(group + 1)

    # ------------------------------------------------------------------ gradient reduce-scatter per microbatch
    def _unit_backward_done(self, group: int) -> None:
        if group in self._launched:
            return
        self._reduce_group(group)
        if group - 1 >= 0:
            # the next group in backward order needs its parameters again ...
            self._need(group - 1)
            # ... and its gradient buffer was last used by the group two places later in backward order: every rank must
            # have finished reading that one before this group's backward writes into the buffer
            self._await_readers(group + 1)
        if group - 2 >= 0:
            self._gather(group - 2)

    def _await_readers(self, group: int) -> None:
        """The compute stream waits until this rank's own reduction and (bounded) every peer's have finished reading this
        rank's gradient buffer of ``group`` in this microbatch."""
        if group >= len(self.groups) or not self.cuda or group not in self._launched:
            return
        cur = torch.cuda.current_stream(self.device)
        ev = self.rs_events.get(group)
        if ev is not None:
            cur.wait_event(ev)
        if self.world > 1:
            for ui in self.groups[group]:
                if self.units[ui].local:
                    continue
                L.check(L.load().dewb_wait_flags(L.ptr(self.flags.tensor), ctypes.c_int(ui * 2 + SLOT_DONE), ctypes.c_int(self.world),
                                                 ctypes.c_uint(self.rs_seq), ctypes.c_ulonglong(self.wait_limit_ns),
                                                 L.ptr(L.status(self.device)), L.stream_ptr()), "wait_flags")
                L.count_launches()

    def _fold_autograd_grads(self, u: Unit) -> None:
        """Gradients that arrived through autograd's ``.grad`` join the unit's buffer; a parameter nothing wrote to in this
        microbatch, and the padding between parameters, read as zero."""
        zero = list(getattr(u, "gaps", ()))
        for n, p in u.params:
            stale = getattr(p, "_dewb_fresh", False)
            if p.grad is not None:
                if stale:
                    p.main_grad.copy_(p.grad)
                else:
                    p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None
            elif stale:
                zero.append(p.main_grad.reshape(-1))
            p._dewb_fresh = False
        if zero:
            torch._foreach_zero_(zero)

    def _reduce_group(self, group: int) -> None:
        self._launched.add(group)
        for ui in self.groups[group]:
            u = self.units[ui]
            self._fold_autograd_grads(u)
            if u.local and self.local_group is not None:
                g = self.grad_slots[group % 2].tensor[u.slot_base:u.slot_base + u.size]
                dist.all_reduce(g, group=self.local_group)
            self._reduce(ui)
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
            self.rs_events[group] = ev

    def _reduce(self, ui: int) -> None:
        u = self.units[ui]
        s, lo = u.shard_size, u.shard_offset
        gbuf = self.grad_slots[self.group_of[ui] % 2]
        base = u.slot_base
        if not self.cuda:
            g_full = gbuf.tensor[base:base + u.size]
            if u.world > 1:
                g = torch.empty(s, dtype=torch.float32)
                dist.reduce_scatter_tensor(g, g_full.contiguous(), group=self.group)
            else:
                g = g_full
            if self.replica_group is not None and not u.local:
                dist.all_reduce(g, group=self.replica_group)
            self.reduced[lo:lo + s].add_(g)
            return
        lib = L.load()
        cur = torch.cuda.current_stream(self.device)
        self.comm_stream.wait_stream(cur)
        own = u.local and self.world > 1
        with torch.cuda.stream(self.comm_stream):
            hyper = (ctypes.c_float * 9)(0, 0, 0, 0, 0, 1, 1, 1, 0)
            rc = lib.dewb_rs_adamw_ag(
                gbuf.own_ptr_array(base * 4) if own else gbuf.ptr_array(base * 4),
                self.shards.own_ptr_array(), self._own_ptrs(self.local_flags) if (own or self.world == 1) else self.flags.ptr_array(),
                L.ptr(self.master[lo:lo + s]), L.ptr(self.m[lo:lo + s]), L.ptr(self.v[lo:lo + s]), L.ptr(None),
                L.ptr(self.reduced[lo:lo + s]), L.ptr(None), L.ptr(None),
                ctypes.c_longlong(u.rank * s), ctypes.c_longlong(s), ctypes.c_longlong(u.decay_end), ctypes.c_int(u.rank),
                ctypes.c_int(u.world), hyper, ctypes.c_uint(self.rs_seq), ctypes.c_int(ui * 2 + SLOT_READY),
                ctypes.c_int(ui * 2 + SLOT_DONE), L.ptr(self.block_counter[ui:ui + 1]), ctypes.c_ulonglong(self.wait_limit_ns),
                ctypes.c_int(3), ctypes.c_int(0), ctypes.c_int(self.comm_blocks), L.ptr(L.status(self.device)),
                ctypes.c_void_p(self.comm_stream.cuda_stream))
            L.check(rc, "rs_accumulate")
            L.count_launches()
            if self.replica_group is not None and not u.local:
                dist.all_reduce(self.reduced[lo:lo + s], group=self.replica_group)      # replicas hold the same shard ranges

    # ------------------------------------------------------------------ the update
    def _update(self, ui: int, clipped: bool) -> None:
        """AdamW on this rank's shard of unit ``ui`` from the accumulated gradient; the new bf16 shard replaces the old one."""
        u = self.units[ui]
        s, lo = u.shard_size, u.shard_offset
        if not self.cuda:
            h = list(self._hyper(u))
            lr, b1, b2, eps, wd, bc1, bc2, gs, ed = h
            coef = gs * (float(self.clip[2]) if clipped else 1.0)
            if clipped and self.t.optimizer.config.skip_nonfinite and not math.isfinite(float(self.clip[0])):
                return
            g = self.reduced[lo:lo + s] * coef
            m, v, p = self.m[lo:lo + s], self.v[lo:lo + s], self.master[lo:lo + s]
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            idx = torch.arange(u.rank * s, (u.rank + 1) * s)
            wdv = torch.where(idx < u.decay_end, torch.tensor(wd), torch.tensor(0.0))
            p.mul_(1 - lr * wdv).addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
            if self.ema is not None:
                self.ema[lo:lo + s].mul_(ed).add_(p, alpha=1 - ed)
            self.shards.tensor[lo:lo + s].copy_(p)
            return
        lib = L.load()
        esz = self.shards.tensor.element_size()
        # a world of one whose "full buffer" is this rank's shard: the kernel's push writes the new bf16 shard in place
        rc = lib.dewb_rs_adamw_ag(
            self.grad_slots[0].own_ptr_array(), self.shards.own_ptr_array(lo * esz), self._own_ptrs(self.local_flags),
            L.ptr(self.master[lo:lo + s]), L.ptr(self.m[lo:lo + s]), L.ptr(self.v[lo:lo + s]),
            L.ptr(self.ema[lo:lo + s] if self.ema is not None else None), L.ptr(self.reduced[lo:lo + s]), L.ptr(None),
            L.ptr(self.clip if clipped else None),
            ctypes.c_longlong(0), ctypes.c_longlong(s), ctypes.c_longlong(max(0, min(s, u.decay_end - u.rank * s))), ctypes.c_int(0),
            ctypes.c_int(1), self._hyper(u), ctypes.c_uint(self.seq + 1), ctypes.c_int(ui * 2), ctypes.c_int(ui * 2 + 1),
            L.ptr(self.block_counter[ui:ui + 1]), ctypes.c_ulonglong(self.wait_limit_ns), ctypes.c_int(2),
            ctypes.c_int(int(self.t.optimizer.config.skip_nonfinite)), ctypes.c_int(self.comm_blocks),
            L.ptr(L.status(self.device)), L.stream_ptr())
        L.check(rc, "adamw_shard")
        L.count_launches()

    def step(self, state: TrainState, batch):
        from ..ops import mx as _mx
        _mx.cache_weights(True) if not _mx._CACHE_ON[0] else None
        _mx.weights_changed()          # whatever changed the weights since the last step (a restore, a reload), quantised copies start afresh
        from ..objectives.base import Aux, Step, pool
        from ..training.trainer import _split_rows, tree_detach
        t = self.t
        obj, cfg = t.objective, t.optimizer.config
        parts = _split_rows(batch, t.microbatches or 1)
        step_key = K.fold_in(state.key, state.step)
        self._lr = float(t.optimizer.schedule(state.step))
        self._count = int(state.opt_state["count"]) + 1
        self._updates = state.updates
        clipped = cfg.clip_grads is not None or cfg.skip_nonfinite
        self._two_phase = clipped
        stats_all, metrics_all, effects = [], {}, {}
        rows_per = next(iter(parts[0].values())).shape[0]
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
                mass_known = mass_known * self.batch_ranks
            else:
                mk = torch.tensor([mass_known], dtype=torch.float64, device=self.device)
                dist.all_reduce(mk, group=self.group)
                if self.replica_group is not None:
                    dist.all_reduce(mk, group=self.replica_group)
                mass_known = float(mk.item()) * self.batch_ranks / (self.world * self.replicas)
        self._grad_scale = 1.0 / max(mass_known, 1e-12)
        self.reduced.zero_()
        first = self.batch_index * rows_per * len(parts)
        every_param = [p for u in self.units for _, p in u.params]
        for i, mb in enumerate(parts):
            self.rs_seq += 1
            self._launched = set()
            self.rs_events = {}
            if i > 0:
                # the previous microbatch's reductions ended with the first unit's: once every peer is done reading that one,
                # all of this rank's gradient buffers are free again (their kernels run in stream order)
                self._await_previous_microbatch()
            for p in every_param:
                p._dewb_fresh = True                  # the first gradient written into each buffer overwrites
            st = Step(step=state.step, key=step_key, ema=None, train=True, first_index=first, device=self.device)
            out = obj.loss(None, mb, st)
            stats, aux = out if isinstance(out, tuple) else (out, Aux())
            total, mass = obj.reduce_loss(stats)
            total.backward()
            for group in reversed(range(len(self.groups))):        # units whose input carries no gradient (the embedding)
                if group not in self._launched:
                    self._reduce_group(group)
            stats_all.append(tree_detach(stats))
            for k, v in aux.metrics.items():
                metrics_all.setdefault(k, []).append(tree_detach(v))
            effects.update(aux.effects)
            first += rows_per
        info: Dict[str, Any] = {"learning_rate": self._lr}
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        if clipped:
            local = self.reduced.pow(2).sum().reshape(1) * (self._grad_scale ** 2)
            if self.world > 1:
                dist.all_reduce(local, group=self.group)
            norm = local.sqrt()
            self.clip[0:1] = local
            self.clip[1:2] = norm
            maxn = cfg.clip_grads
            self.clip[2:3] = torch.where((norm > maxn), maxn / (norm + 1e-6), torch.ones_like(norm)) if maxn else torch.ones_like(norm)
            info["grad_norm"] = self.clip[1].clone()
        for ui in range(len(self.units)):
            self._update(ui, clipped)
        self.seq += 1
        self.resident = [None] * self.n_gather                    # every gathered copy is stale now
        if self.cuda and self.world > 1:
            # peers read this rank's new shard in their next gathers: tell them it is written, and wait for theirs
            lib = L.load()
            L.check(lib.dewb_signal_flags(self.flags.ptr_array(), ctypes.c_int(self.sync_slot), ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                          ctypes.c_uint(self.seq), L.stream_ptr()), "signal_flags")
            L.check(lib.dewb_wait_flags(L.ptr(self.flags.tensor), ctypes.c_int(self.sync_slot), ctypes.c_int(self.world), ctypes.c_uint(self.seq),
                                        ctypes.c_ulonglong(self.wait_limit_ns), L.ptr(L.status(self.device)), L.stream_ptr()), "wait_flags")
            L.count_launches(2)
        elif self.world > 1:
            dist.barrier(group=self.group)
        skipped = bool(clipped and cfg.skip_nonfinite and not math.isfinite(float(self.clip[0])))
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
        metrics = {"loss": pool(stats_all), **{k: pool(v) for k, v in metrics_all.items()}, **info}
        _mx.weights_changed()          # the update just written makes this step's quantised copies stale for whoever runs next
        return new_state, metrics

    def _await_previous_microbatch(self) -> None:
        """Before a microbatch writes gradients again: this rank's reductions of the previous one have run (stream order) and,
        bounded, every peer has finished reading this rank's buffers - their reductions run in stream order too, so the flag
        of the last one (the first group's) covers them all."""
        if not self.cuda:
            return
        torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        if self.world == 1:
            return
        ui = next((i for i in self.groups[0] if not self.units[i].local), None)
        if ui is None:
            return
        L.check(L.load().dewb_wait_flags(L.ptr(self.flags.tensor), ctypes.c_int(ui * 2 + SLOT_DONE), ctypes.c_int(self.world),
                                         ctypes.c_uint(self.rs_seq - 1), ctypes.c_ulonglong(self.wait_limit_ns),
                                         L.ptr(L.status(self.device)), L.stream_ptr()), "wait_flags")
        L.count_launches()

    # ------------------------------------------------------------------ memory accounting
    def state_bytes(self) -> Dict[str, int]:
        """Device bytes this rank holds for parameters, gradients and optimizer state (activations excluded)."""
        esz = self.shards.tensor.element_size()
        return {"param_shards": self.shard_total * esz, "masters_moments": self.shard_total * 12,
                "ema": self.shard_total * 4 if self.ema is not None else 0, "grad_accumulator": self.shard_total * 4,
                "gather_buffers": self.n_gather * self.slot_size * esz, "grad_buffers": 2 * self.slot_size * 4}
