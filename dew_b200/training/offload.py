"""Training with the optimizer state in host memory: the fp32 master weights and both Adam moments live in pinned host
memory and stream through two device slots per update, so a GPU holds only the bf16 compute weights, the gradients and the
activations (2 + 4 bytes per parameter instead of 18).

Per step, after the backward: the parameters are walked in buckets of about ``bucket_bytes``; while bucket i is updated on
the compute stream (``ops.adamw_`` on the slot, which also refreshes the bf16 compute copy), bucket i + 1 is already crossing
host -> device on the copy stream and bucket i - 1 is on its way back.  Global-norm clipping and ``skip_nonfinite`` are
decided before the walk from the gradients alone.  On a CPU-only process the same code runs with the slots as plain tensors.

``Trainer(..., offload="optimizer")`` selects this engine (one device, AdamW / Adam, no EMA).

Reference: the host-offloaded execution of src/dew/training/execution.py / staging.py / streaming.py (state kept on the host
and staged through device buffers around the update).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Mapping, Tuple

import torch

from .. import ops
from ..objectives.base import Aux, Step, pool
from ..utils import keys as K
from ..utils.trees import flatten, unflatten
from .state import TrainState
from .trainer import LocalEngine, _split_rows, tree_detach


class HostOffloadEngine(LocalEngine):
    def __init__(self, trainer, bucket_bytes: int = 256 << 20):
        super().__init__(trainer)
        cfg = trainer.optimizer.config
        if cfg.optimizer not in ("adamw", "adam"):
            raise ValueError(f"optimizer-state offload runs AdamW / Adam; got {cfg.optimizer!r}")
        if cfg.state_dtype != "float32":
            raise ValueError("optimizer-state offload keeps fp32 moments")
        if trainer.objective.ema_spec() is not None:
            raise ValueError("optimizer-state offload does not keep an EMA copy (it would double the host traffic): pass ema_decay=None")
        self.bucket_elems = max(1, bucket_bytes // 4)

    # ------------------------------------------------------------------ state
    def fresh_state(self, key: int) -> TrainState:
        t = self.t
        variables = t.objective.init(K.fold_in(key, "init"))
        live = flatten(variables["params"])
        dev = next(self.model.parameters()).device
        self.device = dev
        pin = dev.type == "cuda"
        # masters and moments on the host; the module keeps the (narrow) compute copies on the device
        masters = {k: _host(v.detach().float(), pin) for k, v in live.items()}
        if t.param_dtype is not None and t.param_dtype != torch.float32:
            with torch.no_grad():
                for p in self.model.parameters():
                    p.data = p.data.to(t.param_dtype)
        from ..utils.trees import module_variables
        self.compute = flatten(module_variables(self.model)["params"])
        variables = {**variables, "params": unflatten(masters)}
        opt_state = {"count": torch.tensor(0, dtype=torch.int64),
                     "mu": unflatten({k: _host(torch.zeros_like(v), pin) for k, v in masters.items()}),
                     "nu": unflatten({k: _host(torch.zeros_like(v), pin) for k, v in masters.items()})}
        self._slots = None
        return TrainState(variables=variables, opt_state=opt_state, ema=None, key=key, scale=None)

    def adopt(self, state: TrainState) -> TrainState:
        pin = self.device.type == "cuda"
        state.variables = {**state.variables, "params": unflatten({k: _host(v.float(), pin) for k, v in flatten(state.variables["params"]).items()})}
        for name in ("mu", "nu"):
            state.opt_state[name] = unflatten({k: _host(v.float(), pin) for k, v in flatten(state.opt_state[name]).items()})
        masters = flatten(state.variables["params"])
        with torch.no_grad():
            for k, c in self.compute.items():
                c.copy_(masters[k].to(c.device))
        return state

    def device_bytes(self) -> Dict[str, int]:
        """What the device holds for the model under this engine (weights + gradients + the streaming slots)."""
        n = sum(c.numel() for c in self.compute.values())
        esz = next(iter(self.compute.values())).element_size()
        slots = 0 if self._slots is None else sum(s.numel() * 4 for pair in self._slots for s in pair)
        return {"weights": n * esz, "gradients": n * 4, "slots": slots, "host_state": n * 12}

    # ------------------------------------------------------------------ the step
    def step(self, state: TrainState, batch: Mapping[str, torch.Tensor]) -> tuple:
        t = self.t
        obj = t.objective
        cfg = t.optimizer.config
        parts = _split_rows(batch, t.microbatches or 1)
        step_key = K.fold_in(state.key, state.step)
        dev = self.device
        for p in self.model.parameters():
            p.grad = None
        stats_all, metrics_all, effects = [], {}, {}
        mass_total = 0.0
        first = 0
        for mb in parts:
            rows = next(iter(mb.values())).shape[0]
            st = Step(step=state.step, key=step_key, ema=None, train=True, first_index=first, device=dev)
            out = obj.loss(None, mb, st)
            stats, aux = out if isinstance(out, tuple) else (out, Aux())
            total, mass = obj.reduce_loss(stats)
            total.backward()
            stats_all.append(tree_detach(stats))
            for k, v in aux.metrics.items():
                metrics_all.setdefault(k, []).append(tree_detach(v))
            effects.update(aux.effects)
            mass_total = mass_total + (mass.detach() if isinstance(mass, torch.Tensor) else mass)
            first += rows
        inv = 1.0 / max(float(mass_total), 1e-12)
        from ..utils.trees import module_path_to_tree_path
        grads = {module_path_to_tree_path(n): p.grad for n, p in self.model.named_parameters() if p.grad is not None}
        sq = torch.zeros((), dtype=torch.float32, device=dev)
        for g in grads.values():
            sq = sq + g.float().pow(2).sum()
        norm = sq.sqrt() * inv
        lr = float(t.optimizer.schedule(state.step))
        info: Dict[str, Any] = {"grad_norm": norm, "learning_rate": lr}
        skipped = bool(cfg.skip_nonfinite and not bool(torch.isfinite(norm)))
        new_opt = state.opt_state
        if skipped:
            info["skipped"] = True
        else:
            coef = inv
            if cfg.clip_grads is not None and float(norm) > cfg.clip_grads:
                coef = coef * cfg.clip_grads / (float(norm) + 1e-6)
            count = int(state.opt_state["count"]) + 1
            self._streamed_update(flatten(state.variables["params"]), flatten(state.opt_state["mu"]), flatten(state.opt_state["nu"]),
                                  grads, count, lr, coef)
            new_opt = {**state.opt_state, "count": torch.tensor(count, dtype=torch.int64)}
            obj.apply_effects(state.variables, effects)
        new_state = state.replace(step=state.step + 1, microstep=state.microstep + len(parts),
                                  updates=state.updates + (0 if skipped else 1), opt_state=new_opt,
                                  consumed={"examples": state.consumed.get("examples", 0) + first,
                                            "tokens": state.consumed.get("tokens", 0) + int(obj.row_tokens(batch) or 0)})
        metrics = {"loss": pool(stats_all), **{k: pool(v) for k, v in metrics_all.items()}, **info}
        return new_state, metrics

    # ------------------------------------------------------------------ the streamed update
    def _buckets(self, masters: Mapping[str, torch.Tensor]) -> List[List[Tuple[str, int, int]]]:
        """Parameters cut into pieces of at most ``bucket_elems`` elements, packed into buckets: (path, first element, count)."""
        buckets, cur, room = [], [], self.bucket_elems
        for path, p in masters.items():
            n, at = p.numel(), 0
            while at < n:
                take = min(n - at, room)
                cur.append((path, at, take))
                at += take
                room -= take
                if room == 0:
                    buckets.append(cur)
                    cur, room = [], self.bucket_elems
        if cur:
            buckets.append(cur)
        return buckets

    def _streamed_update(self, masters, mu, nu, grads, count: int, lr: float, coef: float) -> None:
        cfg = self.t.optimizer.config
        opts = cfg.optimizer_opts
        b1, b2, eps = opts.get("b1", 0.9), opts.get("b2", 0.999), opts.get("eps", 1e-8)
        dev = self.device
        cuda = dev.type == "cuda"
        E = self.bucket_elems
        if self._slots is None:
            self._slots = [tuple(torch.empty(E, dtype=torch.float32, device=dev) for _ in range(3)) for _ in range(2)]
            self._copy_stream = torch.cuda.Stream(device=dev) if cuda else None
        buckets = self._buckets(masters)
        loaded: List[Any] = [None, None]        # events: the slot's host -> device copies are done
        stored: List[Any] = [None, None]        # events: the slot's device -> host copies are done (the slot may be refilled)
        main = torch.cuda.current_stream(dev) if cuda else None

        def load(i: int) -> None:
            slot = self._slots[i % 2]
            if cuda:
                with torch.cuda.stream(self._copy_stream):
                    if stored[i % 2] is not None:
                        self._copy_stream.wait_event(stored[i % 2])
                    at = 0
                    for path, first, n in buckets[i]:
                        for s, src in zip(slot, (masters, mu, nu)):
                            s[at:at + n].copy_(src[path].view(-1)[first:first + n], non_blocking=True)
                        at += n
                    ev = torch.cuda.Event()
                    ev.record(self._copy_stream)
                    loaded[i % 2] = ev
            else:
                at = 0
                for path, first, n in buckets[i]:
                    for s, src in zip(slot, (masters, mu, nu)):
                        s[at:at + n].copy_(src[path].view(-1)[first:first + n])
                    at += n

        if buckets:
            load(0)
        for i, bucket in enumerate(buckets):
            if i + 1 < len(buckets):
                load(i + 1)                                        # the next bucket crosses while this one is updated
            pm, pmu, pnu = self._slots[i % 2]
            if cuda:
                main.wait_event(loaded[i % 2])
            at = 0
            for path, first, n in bucket:
                g = grads.get(path)
                c = self.compute[path]
                if g is not None:
                    scale, wd = self.t.optimizer._group_of(path)
                    wdk = wd if cfg.optimizer == "adamw" else 0.0
                    narrow = c.view(-1)[first:first + n] if (c.dtype == torch.bfloat16 and c.is_contiguous()) else None
                    ops.adamw_(pm[at:at + n], pmu[at:at + n], pnu[at:at + n], g.reshape(-1)[first:first + n], step=count, lr=lr * scale,
                               beta1=b1, beta2=b2, eps=eps, weight_decay=wdk, grad_scale=coef, p_bf16=narrow)
                    if narrow is None:
                        with torch.no_grad():
                            c.view(-1)[first:first + n].copy_(pm[at:at + n])
                at += n
            # back to the host (on the copy stream, after the update)
            if cuda:
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(self._copy_stream):
                    self._copy_stream.wait_event(done)
                    at = 0
                    for path, first, n in bucket:
                        for s, dst in zip((pm, pmu, pnu), (masters, mu, nu)):
                            dst[path].view(-1)[first:first + n].copy_(s[at:at + n], non_blocking=True)
                        at += n
                    ev = torch.cuda.Event()
                    ev.record(self._copy_stream)
                    stored[i % 2] = ev
            else:
                at = 0
                for path, first, n in bucket:
                    for s, dst in zip((pm, pmu, pnu), (masters, mu, nu)):
                        dst[path].view(-1)[first:first + n].copy_(s[at:at + n])
                    at += n
        if cuda:
            main.wait_stream(self._copy_stream)
            self._copy_stream.synchronize()                       # the host tensors are read by the next step's copies and by checkpoints


def _host(x: torch.Tensor, pin: bool) -> torch.Tensor:
    h = x.detach().to("cpu", copy=True).contiguous()
    return h.pin_memory() if pin else h
