"""``Trainer``: the training loop.  Constructing one allocates nothing and opens nothing.

Parity: src/dew/training/trainer.py (``__init__`` :271-386, ``fit`` :1174-1273, ``_training_loop`` :1340-1457) and
src/dew/training/transaction.py (``Transaction.step`` :1766-1884: microbatch loop -> pooled statistics -> clip ->
optimizer -> effects -> EMA -> skip_nonfinite).  The step itself is delegated to an *engine*:

* ``LocalEngine``   one device; fp32 masters and a bf16 compute copy on a GPU, AdamW through the fused flat kernel
* ``FSDPEngine``    (``dew_b200.parallel.fsdp``) sharded masters / moments / EMA with the fused reduce-scatter + AdamW +
                    all-gather kernel, a resident gathered compute copy and full fp32 gradient accumulators
* ``PipelineEngine`` / ``DataParallelEngine`` and the compositions with tensor / expert parallelism:
                    ``dew_b200.parallel.compose.build_engine`` turns ``Trainer(mesh=MeshSpec(...))`` into the engine
"""
from __future__ import annotations

import math
import os
import signal
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, Iterator, List, Mapping, Optional, Sequence, Union

import torch

from ..telemetry.trace import TRACER

from ..objectives.base import Aux, Objective, Ratio, Step, pool
from ..optim import OptimConfig, Optimizer, ema_update
from ..utils import keys as K
from ..utils.trees import flatten, module_variables, tree_map, unflatten
from .state import TrainState
from .tracker import MemoryTracker


@dataclass(frozen=True)
class Cooldown:
    """A learning-rate cooldown window: from step ``at`` the rate falls from 1x to ``floor``x over ``steps`` steps ("linear",
    "cosine" or "sqrt" - one minus the square root of the progress, the WSD recipe) and stays there."""
    at: int
    steps: int
    floor: float = 0.0
    shape: str = "linear"

    def factor(self, step: int) -> float:
        if step < self.at:
            return 1.0
        x = min(1.0, (step - self.at) / max(1, self.steps))
        fall = {"linear": x, "cosine": 0.5 * (1 - math.cos(math.pi * x)), "sqrt": math.sqrt(x)}[self.shape]
        return 1.0 - (1.0 - self.floor) * fall


class Preempted(SystemExit):
    """Raised after a preemption checkpoint; exit status 143 like a SIGTERM'd process."""

    def __init__(self):
        super().__init__(143)


@dataclass
class Plateau:
    """Stop when ``metric`` has not improved by ``min_delta`` for ``patience`` evaluations."""
    metric: str = "loss"
    patience: int = 5
    min_delta: float = 0.0
    mode: str = "min"
    _best: Optional[float] = None
    _bad: int = 0

    def update(self, metrics: Mapping[str, float]) -> bool:
        v = metrics.get(self.metric)
        if v is None:
            return False
        better = self._best is None or (v < self._best - self.min_delta if self.mode == "min" else v > self._best + self.min_delta)
        if better:
            self._best, self._bad = v, 0
        else:
            self._bad += 1
        return self._bad >= self.patience


@dataclass(frozen=True)
class Pause:
    """End the run once it has trained ``fraction`` of its budget, its state and data position written in full, so a run
    resumed from that checkpoint trains on as one that never paused (the budget still sizes the schedule).  Resume without it,
    or with a later fraction, to go on.  Reference: src/dew/training/budget.py:123-160."""
    fraction: float

    def __post_init__(self):
        if not 0 < self.fraction < 1:
            raise ValueError(f"Pause needs a fraction of the budget in (0, 1), got {self.fraction}")

    def at(self, steps: int) -> int:
        """The step a run of ``steps`` pauses at: the whole update nearest the fraction; a pause before the first update or
        at the budget's end is refused (the run would not start, or ends there anyway)."""
        step = round(self.fraction * steps)
        if step <= 0 or step >= steps:
            raise ValueError(f"a pause at {self.fraction} of {steps} steps falls on step {step}: before the first update or at the end")
        return step


@dataclass
class Best:
    """Track the best value of a metric (used with ``Checkpoints(ranking=...)`` and ``restore_best``)."""
    metric: str = "loss"
    mode: str = "min"


@dataclass
class Evaluation:
    data: Any
    every: Optional[int] = None
    steps: Optional[int] = None
    name: str = "val"


@dataclass
class ProfileWindow:
    """Capture ``steps`` training steps starting at ``start`` with torch.profiler and report device time."""
    start: int = 10
    steps: int = 3
    directory: Optional[str] = None


def _split_rows(batch: Mapping[str, torch.Tensor], parts: int) -> List[Dict[str, torch.Tensor]]:
    if parts <= 1:
        return [dict(batch)]
    rows = next(iter(batch.values())).shape[0]
    if rows % parts:
        raise ValueError(f"a batch of {rows} rows does not split into {parts} microbatches")
    n = rows // parts
    return [{k: (v[i * n:(i + 1) * n] if isinstance(v, torch.Tensor) and v.shape[:1] == (rows,) else v)
             for k, v in batch.items()} for i in range(parts)]


class LocalEngine:
    """Single-device step.  On a GPU with ``param_dtype=bfloat16`` the model runs on bf16 compute copies while
    ``state.variables`` holds the fp32 masters; gradients accumulate in fp32."""

    def __init__(self, trainer: "Trainer"):
        self.t = trainer
        self.model = trainer.objective.model
        self.masters: Optional[Dict[str, torch.Tensor]] = None

    def fresh_state(self, key: int) -> TrainState:
        t = self.t
        variables = t.objective.init(K.fold_in(key, "init"))
        live = flatten(variables["params"])
        narrow = t.param_dtype is not None and any(p.dtype != torch.float32 for p in live.values())
        if t.param_dtype is not None and t.param_dtype != torch.float32:
            # masters are fp32 copies; the module keeps the narrow compute copies
            masters = {k: v.detach().float().clone() for k, v in live.items()}
            with torch.no_grad():
                for p in self.model.parameters():
                    p.data = p.data.to(t.param_dtype)
            self.compute = flatten(module_variables(self.model)["params"])
            variables = {**variables, "params": unflatten(masters)}
        else:
            self.compute = None
        opt_state = t.optimizer.init(variables["params"])
        spec = t.objective.ema_spec()
        ema = None
        if spec is not None:
            ema = {"params": tree_map(lambda x: x.detach().clone(), variables["params"])}
        scale = None
        if t.dynamic_scale:
            # loss scaling for narrow gradients: the loss is multiplied by `scale` before backward and the gradients divided by
            # it; a step with a non-finite gradient is dropped and halves the scale, `growth_interval` good steps double it
            scale = {"scale": torch.tensor(float(2 ** 15)), "good_steps": torch.tensor(0, dtype=torch.int64)}
        return TrainState(variables=variables, opt_state=opt_state, ema=ema, key=key, scale=scale)

    def adopt(self, state: TrainState) -> TrainState:
        """Bind a restored state: the module's parameters take the state's values."""
        live = dict(self.model.named_parameters())
        from ..utils.trees import variables_for_call
        flat = variables_for_call(self.model, state.variables)
        with torch.no_grad():
            for n, p in live.items():
                if n in flat:
                    p.copy_(flat[n].to(p.dtype))
        if self.t.param_dtype in (None, torch.float32):
            # masters alias the module parameters again
            state.variables = {**state.variables, **module_variables(self.model)}
        return state

    def step(self, state: TrainState, batch: Mapping[str, torch.Tensor]) -> tuple:
        t = self.t
        obj = t.objective
        parts = _split_rows(batch, t.microbatches or 1)
        step_key = K.fold_in(state.key, state.step)
        dev = next(self.model.parameters()).device
        for p in self.model.parameters():
            p.grad = None
        stats_all, metrics_all, effects = [], {}, {}
        mass_total = 0.0
        first = 0
        model_vars = None if self.compute is not None else state.variables
        for mb in parts:
            rows = next(iter(mb.values())).shape[0]
            st = Step(step=state.step, key=step_key, ema=state.ema, train=True, first_index=first, device=dev)
            out = obj.loss(model_vars, mb, st)
            stats, aux = out if isinstance(out, tuple) else (out, Aux())
            total, mass = obj.reduce_loss(stats)
            scale = float(state.scale["scale"]) if state.scale else 1.0
            (total * scale).backward()
            stats_all.append(tree_detach(stats))
            for k, v in aux.metrics.items():
                metrics_all.setdefault(k, []).append(tree_detach(v))
            effects.update(aux.effects)
            mass_total = mass_total + (mass.detach() if isinstance(mass, torch.Tensor) else mass)
            first += rows
        pooled = pool(stats_all)
        mass_f = float(mass_total)
        sync = getattr(self, "grad_sync", None)
        if sync is not None:
            mass_f = sync(list(self.model.parameters()), mass_f)        # data parallelism: gradients and mass summed over the ranks
        inv = 1.0 / max(mass_f, 1e-12)
        if state.scale:
            inv /= float(state.scale["scale"])
        grads = {}
        from ..utils.trees import module_path_to_tree_path
        for n, p in self.model.named_parameters():
            if p.grad is not None:
                grads[module_path_to_tree_path(n)] = p.grad
        new_opt, info = t.optimizer.update(state.variables["params"], unflatten(grads), state.opt_state,
                                           state.step, grad_scale=inv)
        skipped = bool(info.get("skipped", False))
        new_scale = state.scale
        if state.scale:
            cur, good = float(state.scale["scale"]), int(state.scale["good_steps"])
            if skipped:
                cur, good = max(cur * 0.5, 1.0), 0
            else:
                good += 1
                if good >= t.scale_growth_interval:
                    cur, good = min(cur * 2.0, float(2 ** 24)), 0
            new_scale = {"scale": torch.tensor(cur), "good_steps": torch.tensor(good, dtype=torch.int64)}
            info["loss_scale"] = cur
        if not skipped and self.compute is not None:
            masters = flatten(state.variables["params"])
            with torch.no_grad():
                for k, c in self.compute.items():
                    c.copy_(masters[k])
        if not skipped:
            obj.apply_effects(state.variables, effects)
        spec = obj.ema_spec()
        ema = state.ema
        if ema is not None and not skipped:
            decay = spec.at(state.updates + 1)
            ema_update(ema["params"], state.variables["params"], decay)
        rows_total = first
        new_state = state.replace(step=state.step + 1, microstep=state.microstep + len(parts),
                                  updates=state.updates + (0 if skipped else 1), opt_state=new_opt, ema=ema, scale=new_scale,
                                  consumed={"examples": state.consumed.get("examples", 0) + rows_total,
                                            "tokens": state.consumed.get("tokens", 0) + int(obj.row_tokens(batch) or 0)})
        metrics = {"loss": pooled, **{k: pool(v) for k, v in metrics_all.items()}, **info}
        return new_state, metrics


def tree_detach(x):
    if isinstance(x, torch.Tensor):
        return x.detach()
    if hasattr(x, "__dataclass_fields__"):
        return type(x)(**{f: tree_detach(getattr(x, f)) for f in x.__dataclass_fields__})
    return x


class Trainer:
    def __init__(self, objective: Objective, optimizer: Union[OptimConfig, Optimizer, None] = None, *, key: int = 0,
                 mesh=None, layout=None, microbatches: Optional[int] = None, accumulation: int = 1, split=None,
                 dynamic_scale: bool = False, checkpoints=None, tracker=None, step=None, profile: Optional[ProfileWindow] = None,
                 param_dtype: Optional[torch.dtype] = None, diloco=None, data_resume: str = "relaxed",
                 skip_nonfinite: bool = False, record: bool = False, tune_kernels: bool = False, offload: Optional[str] = None):
        self.objective = objective
        if optimizer is None:
            optimizer = OptimConfig()
        if isinstance(optimizer, OptimConfig):
            if skip_nonfinite:
                optimizer.skip_nonfinite = True
            optimizer = optimizer.build()
        self.optimizer = objective.optimizer(optimizer)
        self.key = K.key(key)
        self.mesh, self.layout = mesh, layout
        self.microbatches = microbatches if microbatches is not None else (accumulation if accumulation > 1 else None)
        self.dynamic_scale = dynamic_scale
        self.scale_growth_interval = 2000
        if dynamic_scale:
            self.optimizer.config.skip_nonfinite = True      # an overflowed step must be dropped, not applied
        if tune_kernels:
            from ..ops import tuning
            tuning.enable(True)
        self.tune_kernels = tune_kernels
        if offload not in (None, "optimizer"):
            raise ValueError(f"offload must be None or 'optimizer', not {offload!r}")
        self.offload = offload          # 'optimizer': fp32 masters and Adam moments in pinned host memory, streamed through device slots
        self._diloco_runner = None
        self.checkpoints, self.tracker = checkpoints, tracker
        self.custom_step = step
        self.profile = profile
        self.param_dtype = param_dtype
        self.diloco = diloco
        self.data_resume = data_resume
        self.skip_nonfinite = skip_nonfinite
        self.record = record
        self._engine = None
        self._preempted = False
        self.history: List[Dict[str, Any]] = []

    # ------------------------------------------------------------------ engine / state
    def engine(self):
        """The engine the mesh asks for, built once: every axis of ``MeshSpec`` (fsdp, data / replicas, tensor, expert, stage)
        is composed by ``dew_b200.parallel.compose.build_engine``; without a mesh, or on one process, the local engine."""
        if self._engine is None:
            from ..parallel.compose import build_engine
            self._engine = build_engine(self)
        return self._engine

    def _fresh_state(self) -> TrainState:
        return self.engine().fresh_state(self.key)

    def place(self, state: Optional[TrainState] = None) -> TrainState:
        return self.engine().adopt(state) if state is not None else self._fresh_state()

    def validate(self, devices: int = 1, memory_bytes: float = 180e9) -> Dict[str, Any]:
        """Dry-run placement report on the host: bytes per device and implied collectives, without allocating
        device memory (reference: Trainer.validate, src/dew/training/trainer.py:666)."""
        from ..parallel.layout import Layout, placement_report
        return placement_report(self.objective.model, self.mesh, self.layout or Layout(), devices, memory_bytes,
                                state_dtype=self.optimizer.config.state_dtype, ema=self.objective.ema_spec() is not None)

    def compile(self, batch: Optional[Mapping[str, torch.Tensor]] = None):
        """Warm the kernels / allocator on one batch shape (there is no tracing compiler to run)."""
        return self

    # ------------------------------------------------------------------ fit
    def fit(self, dataset, *, state: Optional[TrainState] = None, resume: str = "auto", steps: Optional[int] = None,
            epochs: Optional[int] = None, tokens: Optional[int] = None, examples: Optional[int] = None,
            log_every: int = 100, eval_every: Optional[int] = None, checkpoint_every: Optional[Union[int, str]] = None,
            checkpoint_final: bool = True, metrics: Sequence[Any] = (), preview: Optional[int] = None,
            best: Optional[Best] = None, stop: Optional[Plateau] = None, validation=None, restore_best: bool = False,
            observe: Optional[Callable] = None, device_prefetch: int = 0, cooldowns: Sequence["Cooldown"] = (),
            summaries: Optional[Callable[[TrainState], Dict[str, float]]] = None, pause: Optional[Pause] = None) -> TrainState:
        """``cooldowns``: learning-rate cooldown windows applied on top of the optimizer's schedule for this fit (branching a
        decayed run off a constant-rate trunk); ``summaries``: a callable whose scalars are logged beside the loss at the
        logging cadence (weight norms, router statistics, ...)."""
        eng = self.engine()
        base_schedule = self.optimizer.schedule
        if cooldowns:
            self.optimizer.schedule = lambda step: base_schedule(step) * math.prod(c.factor(step) for c in cooldowns)
        it, loader = _iterate(dataset)
        start_step = None
        if state is None:
            if self.checkpoints is not None and resume != "never":
                start_step = self.checkpoints.resumed(resume)
            state = eng.fresh_state(self.key)
            if start_step is not None:
                if hasattr(eng, "import_state"):
                    # sharded engines read the layout-free checkpoint and keep the slices of their own shards
                    state = eng.import_state(self.checkpoints.restore(None, start_step), state)
                else:
                    state = eng.adopt(self.checkpoints.restore(state, start_step))
                pos = state.deferred
                if pos is not None and hasattr(loader, "restore"):
                    loader.restore(pos)
                    it = iter(loader)
                elif pos is not None and self.data_resume == "strict":
                    raise RuntimeError("data_resume='strict' but the dataset cannot restore a position")
        else:
            state = eng.adopt(state)
        target = _target_steps(steps, epochs, tokens, examples, loader, self.objective)
        every = _every(checkpoint_every, target)
        if pause is not None:
            target = pause.at(target)           # cadences above stay those of the whole budget; the final checkpoint is the pause's
        self._install_preemption()
        tracker = self.tracker
        window: List[Dict[str, Any]] = []
        t_last = time.perf_counter()
        stop_now = False
        prof = None
        while state.step < target and not stop_now:
            try:
                batch = next(it)
            except StopIteration:
                if epochs is None and steps is not None and hasattr(loader, "__iter__"):
                    it = iter(loader)
                    try:
                        batch = next(it)
                    except StopIteration:
                        break
                else:
                    break
            batch = _to_device(batch, self.objective.model)
            if self.profile is not None and state.step == self.profile.start:
                prof = torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU] + (
                    [torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else []))
                prof.__enter__()
            if self.custom_step is not None:
                state, m = self.custom_step(self, state, batch)
            else:
                with TRACER.span("train_step", step=state.step):
                    state, m = eng.step(state, batch)
            if prof is not None and state.step >= self.profile.start + self.profile.steps:
                prof.__exit__(None, None, None)
                self.profile_report = prof.key_averages().table(row_limit=20)
                if self.profile.directory:
                    os.makedirs(self.profile.directory, exist_ok=True)
                    prof.export_chrome_trace(os.path.join(self.profile.directory, f"trace_{state.step}.json"))
                prof = None
            if self.diloco is not None:
                self._diloco_step(state)
            window.append(m)
            if observe is not None:
                observe(state, m)
            if state.step % log_every == 0 or state.step == target:
                now = time.perf_counter()
                row = _summarise(window)
                row["step_time_ms"] = 1000 * (now - t_last) / max(1, len(window))
                rows = next(iter(batch.values())).shape[0]
                row["samples_per_sec"] = rows * len(window) / max(now - t_last, 1e-9)
                t_last, window = now, []
                if summaries is not None:
                    row.update({k: float(v) for k, v in summaries(state).items()})
                self.history.append({"step": state.step, **row})
                if tracker is not None:
                    tracker.log(state.step, row)
            if validation is not None and eval_every and state.step % eval_every == 0:
                ev = self.evaluate(state, validation)
                self.history.append({"step": state.step, **{f"val/{k}": v for k, v in ev.items()}})
                if tracker is not None:
                    tracker.log(state.step, {f"val/{k}": v for k, v in ev.items()})
                if stop is not None and stop.update(ev):
                    stop_now = True
            if preview and state.step % preview == 0 and tracker is not None:
                art = self.objective.preview(state.averaged, batch, key=K.fold_in(self.key, state.step))
                if art is not None:
                    tracker.artifact(state.step, "preview", art)
            if self.checkpoints is not None and every and state.step % every == 0 and state.step < target:
                self._save(state, loader)
            if self._preempted:
                if self.checkpoints is not None:
                    self._save(state, loader)
                    self.checkpoints.wait()
                raise Preempted()
        if self.checkpoints is not None and checkpoint_final:
            self._save(state, loader)
            self.checkpoints.wait()
        if restore_best and self.checkpoints is not None and self.checkpoints.best() is not None:
            state = eng.adopt(self.checkpoints.restore(state, self.checkpoints.best()))
        self.optimizer.schedule = base_schedule
        return state

    def _diloco_step(self, state: TrainState) -> None:
        """DiLoCo: after every `every` inner steps the replicas along the mesh's ``diloco`` axis average how far they moved
        and apply it with the outer optimizer; the compute copies are refreshed from the new masters."""
        from ..parallel.diloco import DiLoCo, DiLoCoConfig
        if self._diloco_runner is None:
            cfg = self.diloco if isinstance(self.diloco, DiLoCoConfig) else DiLoCoConfig(**dict(self.diloco)) if isinstance(self.diloco, Mapping) else DiLoCoConfig()
            eng = self.engine()
            if hasattr(eng, "master"):
                masters = [eng.master]                                   # the sharded engine's flat fp32 shard
            else:
                masters = [v for v in flatten(state.variables["params"]).values() if v.dtype.is_floating_point]
            group = None
            mesh = getattr(eng, "mesh", None)
            if mesh is not None:
                group = mesh.group("diloco")
            self._diloco_runner = DiLoCo(masters, cfg, group=group)
        if self._diloco_runner.after_inner_step():
            eng = self.engine()
            if hasattr(eng, "refresh_compute_copy"):
                eng.refresh_compute_copy()
            elif getattr(eng, "compute", None) is not None:
                masters = flatten(state.variables["params"])
                with torch.no_grad():
                    for k, c in eng.compute.items():
                        c.copy_(masters[k])

    def _save(self, state: TrainState, loader) -> None:
        pos = loader.position() if hasattr(loader, "position") else None
        last = next((h for h in reversed(self.history) if "loss" in h), {})
        m = {k: v for k, v in last.items() if isinstance(v, (int, float)) and k != "step"}
        eng = self.engine()
        if hasattr(eng, "export_state"):
            state = eng.export_state(state)            # collective; whole trees on rank 0, None elsewhere
            if state is None:
                return
        self.checkpoints.save(state.step, state, saved=pos, metrics=m)

    def evaluate(self, state: TrainState, data, steps: Optional[int] = None) -> Dict[str, float]:
        it, _ = _iterate(data)
        acc: Dict[str, List[Any]] = {}
        dev = next(self.objective.model.parameters()).device
        for i, batch in enumerate(it):
            if steps is not None and i >= steps:
                break
            batch = _to_device(batch, self.objective.model)
            out = self.objective.evaluate(state.averaged if state.ema is not None else None, batch,
                                          Step(step=state.step, key=K.fold_in(K.fold_in(self.key, "eval"), i), train=False, device=dev))
            for k, v in out.items():
                acc.setdefault(k, []).append(v)
        return {k: float(pool(v).value()) for k, v in acc.items() if v and hasattr(v[0], "value")}

    def _install_preemption(self) -> None:
        def handler(signum, frame):
            self._preempted = True
        try:
            signal.signal(signal.SIGTERM, handler)
        except ValueError:
            pass  # not the main thread


def _summarise(window: Sequence[Mapping[str, Any]]) -> Dict[str, float]:
    out: Dict[str, float] = {}
    keys = set().union(*[set(m) for m in window])
    for k in keys:
        vals = [m[k] for m in window if k in m]
        if hasattr(vals[0], "value") and hasattr(vals[0], "__add__"):
            out[k] = float(pool(vals).value())
        elif isinstance(vals[0], torch.Tensor):
            out[k] = float(torch.stack([v.float() for v in vals]).mean())
        elif isinstance(vals[0], (int, float)) and not isinstance(vals[0], bool):
            out[k] = float(sum(vals) / len(vals))
    return out


def _iterate(dataset):
    if hasattr(dataset, "train") and callable(getattr(dataset, "train")):
        loader = dataset
        return iter(loader), loader
    return iter(dataset), dataset


def _to_device(batch, model):
    p = next(model.parameters(), None)
    if p is None or not isinstance(batch, Mapping):
        return batch
    return {k: (v.to(p.device, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}


def _target_steps(steps, epochs, tokens, examples, loader, objective) -> int:
    given = [x is not None for x in (steps, epochs, tokens, examples)]
    if sum(given) == 0:
        raise ValueError("fit needs one of steps=, epochs=, tokens=, examples=")
    if steps is not None:
        return int(steps)
    per = getattr(loader, "batch", None)
    if epochs is not None:
        n = getattr(loader, "steps_per_epoch", None)
        if n is None:
            raise ValueError("epochs= needs a dataset that knows its steps_per_epoch")
        return int(epochs * n)
    if examples is not None:
        if per is None:
            raise ValueError("examples= needs a dataset that declares its batch size")
        return int(math.ceil(examples / per))
    row = getattr(loader, "seq_len", None)
    if per is None or row is None:
        raise ValueError("tokens= needs a dataset that declares batch and seq_len")
    return int(math.ceil(tokens / (per * row)))


def _every(value, target: int) -> Optional[int]:
    if value is None:
        return None
    if isinstance(value, str) and value.endswith("%"):
        return max(1, int(target * float(value[:-1]) / 100))
    return int(value)
