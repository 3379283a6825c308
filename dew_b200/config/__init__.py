"""Run configuration: plain dataclasses, ``--set path=value`` overrides, registries for models / objectives, sweeps, and
the ``run.json`` record a checkpoint directory carries so that ``pipeline(dir)`` can rebuild the task.

Parity: src/dew/config/__init__.py (``RunConfig`` :706, ``ObjectiveConfig`` :116, ``_set_arguments`` :410, ``_model_changes``
:469), src/dew/config/trainer.py (``TrainerConfig`` :142-379), src/dew/config/lm.py (``LMRunConfig`` :178),
src/dew/config/diffusion.py, src/dew/config/sweep.py.  Unknown names and fields raise.
"""
from __future__ import annotations

import copy
import dataclasses
import itertools
import json
from dataclasses import dataclass, field, fields, is_dataclass
from typing import Any, Dict, Iterator, List, Mapping, Optional, Sequence, Tuple, Union

from ..utils.registry import lookup


@dataclass
class MeshConfig:
    fsdp: int = 1
    expert: int = 1
    tensor: int = 1
    sequence: int = 1
    stage: int = 1
    replicas: int = 1
    diloco: int = 1


@dataclass
class OptimizerConfig:
    optimizer: str = "adamw"
    learning_rate: float = 3e-4
    schedule: Optional[str] = None          # cosine | linear | wsd | power | onecycle | exponential
    warmup: int = 0
    weight_decay: float = 1e-4
    clip_grads: Optional[float] = None
    state_dtype: str = "float32"
    b1: float = 0.9
    b2: float = 0.999


@dataclass
class TrainerConfig:
    name: str = "run"
    checkpoint_dir: Optional[str] = None
    keep: int = 1
    resume: str = "auto"
    data_resume: str = "relaxed"
    skip_nonfinite: bool = False
    key: int = 0
    steps: Optional[int] = None
    epochs: Optional[int] = None
    tokens: Optional[int] = None
    examples: Optional[int] = None
    log_every: int = 100
    eval_every: Optional[int] = None
    checkpoint_every: Optional[Union[int, str]] = None
    checkpoint_final: bool = True
    accumulation: int = 1
    microbatches: Optional[int] = None
    dynamic_scale: bool = False
    precision: str = "bfloat16"
    mesh: MeshConfig = field(default_factory=MeshConfig)
    profile: Optional[int] = None
    local_directory: Optional[str] = None
    tune_kernels: bool = False


@dataclass
class ModelConfig:
    name: str = "causal_transformer"
    fields: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ObjectiveConfig:
    name: str = "lm"
    options: Dict[str, Any] = field(default_factory=dict)


@dataclass
class DataConfig:
    source: str = "synthetic"          # synthetic (token ids) | synthetic_images | token_files
    image_shape: Tuple[int, int, int] = (32, 32, 3)
    path: Optional[str] = None
    batch: int = 8
    seq_len: int = 128
    workers: int = 0
    seed: int = 0


@dataclass
class RunConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    objective: ObjectiveConfig = field(default_factory=ObjectiveConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    data: DataConfig = field(default_factory=DataConfig)
    tokenizer: Optional[str] = None

    # ------------------------------------------------------------------ record
    def to_record(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    @classmethod
    def from_record(cls, record: Mapping[str, Any]) -> "RunConfig":
        return _build(cls, record)

    def save(self, path) -> None:
        with open(path, "w") as f:
            json.dump(self.to_record(), f, indent=1, sort_keys=True)

    def changes(self, other: "RunConfig", section: str = "model") -> Dict[str, Tuple[Any, Any]]:
        """Fields of ``section`` that differ between this config and ``other`` (the resume-time model diff)."""
        a, b = _flat(getattr(self, section)), _flat(getattr(other, section))
        return {k: (a.get(k), b.get(k)) for k in sorted(set(a) | set(b)) if a.get(k) != b.get(k)}


LMRunConfig = RunConfig


def _build(cls, record: Mapping[str, Any]):
    kwargs = {}
    names = {f.name: f for f in fields(cls)}
    for k, v in record.items():
        if k not in names:
            raise KeyError(f"{cls.__name__} has no field {k!r}; fields: {sorted(names)}")
        ft = names[k].default_factory() if names[k].default_factory is not dataclasses.MISSING else None  # type: ignore
        kwargs[k] = _build(type(ft), v) if is_dataclass(ft) and isinstance(v, Mapping) else v
    return cls(**kwargs)


def _flat(obj, prefix="") -> Dict[str, Any]:
    out = {}
    items = dataclasses.asdict(obj).items() if is_dataclass(obj) else obj.items()
    for k, v in items:
        p = f"{prefix}.{k}" if prefix else k
        if isinstance(v, Mapping):
            out.update(_flat(v, p))
        else:
            out[p] = v
    return out


def _parse(text: str) -> Any:
    try:
        return json.loads(text)
    except json.JSONDecodeError:
        low = text.lower()
        if low in ("none", "null"):
            return None
        if low in ("true", "false"):
            return low == "true"
        return text


def set_path(config: Any, path: str, value: Any) -> None:
    """``set_path(cfg, "trainer.mesh.fsdp", 8)``; dict-valued fields accept new keys, dataclass fields must exist."""
    parts = path.split(".")
    node = config
    for i, part in enumerate(parts[:-1]):
        node = node[part] if isinstance(node, dict) else _field(node, part, ".".join(parts[: i + 1]))
    last = parts[-1]
    if isinstance(node, dict):
        node[last] = value
    else:
        _field(node, last, path)
        setattr(node, last, value)


def _field(node, name, full):
    if not hasattr(node, name):
        known = [f.name for f in fields(node)] if is_dataclass(node) else dir(node)
        raise KeyError(f"unknown configuration path {full!r}; {type(node).__name__} has {known}")
    return getattr(node, name)


def apply_overrides(config: Any, assignments: Sequence[str]) -> Any:
    for a in assignments:
        if "=" not in a:
            raise ValueError(f"--set expects path=value, got {a!r}")
        path, text = a.split("=", 1)
        set_path(config, path.strip(), _parse(text.strip()))
    return config


def sweep(base: RunConfig, grid: Mapping[str, Sequence[Any]]) -> Iterator[RunConfig]:
    """Cartesian product of ``path -> values``; every point is an independent copy named after its overrides."""
    keys = list(grid)
    for combo in itertools.product(*(grid[k] for k in keys)):
        cfg = copy.deepcopy(base)
        for k, v in zip(keys, combo):
            set_path(cfg, k, v)
        cfg.trainer.name = base.trainer.name + "-" + "-".join(f"{k.split('.')[-1]}{v}" for k, v in zip(keys, combo))
        yield cfg


# ------------------------------------------------------------------------------------------------ building a run
def build(config: RunConfig, device=None):
    """(trainer, dataset) from a config: the model and objective come from the registries."""
    import torch

    from .. import data as D
    from ..checkpoints import Checkpoints
    from ..checkpoints.state_trees import leaf_kinds
    from ..optim import OptimConfig, schedules
    from ..parallel.mesh import MeshSpec
    from ..training import ConsoleTracker, LocalTracker, Trackers, Trainer
    from ..models import causal_transformer, dit  # noqa: F401  (registers the built-in models)
    model_cls = lookup(config.model.name, "model")
    model = model_cls(**config.model.fields)
    if device is not None:
        model = model.to(device)
    oc, tc, dc = config.optimizer, config.trainer, config.data
    steps = tc.steps or 1000
    lr: Any = oc.learning_rate
    if oc.schedule:
        lr = {"cosine": schedules.Cosine(oc.learning_rate, steps, oc.warmup), "linear": schedules.Linear(oc.learning_rate, steps, oc.warmup),
              "wsd": schedules.WSD(oc.learning_rate, steps, oc.warmup, decay=max(1, steps // 10)),
              "power": schedules.Power(oc.learning_rate, warmup=oc.warmup), "onecycle": schedules.OneCycle(oc.learning_rate, steps),
              "exponential": schedules.Exponential(oc.learning_rate, warmup=oc.warmup)}[oc.schedule]
    optim = OptimConfig(optimizer=oc.optimizer, learning_rate=lr, weight_decay=oc.weight_decay, clip_grads=oc.clip_grads,
                        state_dtype=oc.state_dtype, optimizer_opts={"b1": oc.b1, "b2": oc.b2})
    tokenizer = D.ByteTokenizer() if config.tokenizer == "byte" else None
    if config.objective.name == "lm":
        from ..objectives.lm import LMObjective
        objective = LMObjective(model, dc.seq_len, tokenizer=tokenizer, **config.objective.options)
    elif config.objective.name == "diffusion":
        from ..objectives.diffusion import DiffusionObjective
        from .. import Field, InputSpec
        from ..diffusion import presets
        opts = dict(config.objective.options)
        process = opts.pop("process", "edm")
        process = {"edm": presets.EDM(regime="pixel"), "flow": presets.Flow()}[process] if isinstance(process, str) else process
        objective = DiffusionObjective(model, process, InputSpec(Field("sample", tuple(dc.image_shape))), **opts)
    else:
        objective = lookup(config.objective.name, "objective")(model, **config.objective.options)
    ckpt = None
    if tc.checkpoint_dir:
        ckpt = Checkpoints(tc.checkpoint_dir, keep=tc.keep, local_directory=tc.local_directory, kinds=leaf_kinds(model))
        ckpt.write_run(config.to_record())
    m = tc.mesh
    mesh = MeshSpec(fsdp=m.fsdp, expert=m.expert, tensor=m.tensor, sequence=m.sequence, stage=m.stage, replicas=m.replicas, diloco=m.diloco)
    trainer = Trainer(objective, optim, key=tc.key, mesh=mesh, microbatches=tc.microbatches, accumulation=tc.accumulation,
                      checkpoints=ckpt, tracker=(Trackers(LocalTracker(tc.checkpoint_dir + "/logs", tc.name), ConsoleTracker(tc.steps)) if tc.checkpoint_dir
                               else ConsoleTracker(tc.steps)),
                      skip_nonfinite=tc.skip_nonfinite, data_resume=tc.data_resume,
                      param_dtype=None if (device is None or str(device) == "cpu") else getattr(torch, tc.precision))
    if dc.source == "synthetic":
        vocab = getattr(model, "vocab_size", 256)
        g = torch.Generator().manual_seed(dc.seed)
        rows = torch.randint(0, vocab, (max(64, dc.batch * 8), dc.seq_len + 1), generator=g)
        dataset = D.Memory({"tokens": rows}).shuffle(dc.seed).repeat().batched(dc.batch)
        dataset.seq_len = dc.seq_len
    elif dc.source == "synthetic_images":
        g = torch.Generator().manual_seed(dc.seed)
        images = torch.rand(max(64, dc.batch * 8), *dc.image_shape, generator=g) * 2 - 1
        dataset = D.Memory({"sample": images}).shuffle(dc.seed).repeat().batched(dc.batch)
    elif dc.source == "token_files":
        dataset = D.TokenFiles(dc.path).shuffle(dc.seed).repeat().pipe(D.presets.token_windows, seq_len=dc.seq_len, batch=dc.batch).workers(dc.workers)
    else:
        raise ValueError(f"unknown data source {dc.source!r}; known: synthetic, synthetic_images, token_files")
    return trainer, dataset
