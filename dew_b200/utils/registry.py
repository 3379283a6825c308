"""Short names for the classes a run is made of, and the records that rebuild them.

A **record** names a class by its import path and carries the fields it was built with::

    {"class": "dew_b200.models.causal_transformer:CausalTransformer", "fields": {"vocab_size": 32000, ...}}
    {"function": "dew_b200.optim.schedules:cosine"}

``to_record(obj)`` writes one (dataclasses and objects that keep their constructor arguments), ``from_record(record)``
imports the module and calls the class with the fields, each converted to the type its annotation declares (nested
records, tuples, optionals, dtypes by name).  So a record loads in a process that imported nothing beforehand, and a class
outside this package needs nothing to be recorded but must live in a package the process trusts (``trust_sources``).
Where a person writes a record - a config file, ``--set`` on the command line - the class may be a short **alias**
(``{"class": "causal_transformer"}``): every kind (models, objectives, optimizers, schedules, mixers, solvers, datasets,
tokenizers) has one table of aliases; the package's own classes are static entries imported only when read, and
``@register("name", kind)`` adds a user's.  Unknown names and unknown fields raise, listing what is known.

Reference: src/dew/registry.py (``Aliases``, ``to_record`` / ``from_record``, ``import_trusted``, "unknown names / fields
raise" of docs/design/api.md:43-52).
"""
from __future__ import annotations

import dataclasses
import enum
import importlib
import inspect
import types
import typing
from typing import Any, Callable, Dict, Iterator, Mapping, Optional, Sequence, Tuple, Union

KINDS = ("model", "objective", "optimizer", "schedule", "mixer", "solver", "dataset", "tokenizer", "run")

# static entries: alias -> import path, imported only when looked up
_STATIC: Dict[str, Dict[str, str]] = {
    "model": {
        "causal_transformer": "dew_b200.models.causal_transformer:CausalTransformer",
        "simple_dit": "dew_b200.models.dit:SimpleDiT",
        "unet": "dew_b200.models.diffusion_backbones:UNet", "uvit": "dew_b200.models.diffusion_backbones:UViT",
        "simple_udit": "dew_b200.models.diffusion_backbones:SimpleUDiT", "simple_mmdit": "dew_b200.models.diffusion_backbones:SimpleMMDiT",
        "video_dit": "dew_b200.models.diffusion_backbones:VideoDiT", "hybrid_dit": "dew_b200.models.diffusion_backbones:HybridDiT",
        "unet_3d": "dew_b200.models.diffusion_backbones:UNet3D", "hierarchical_mmdit": "dew_b200.models.diffusion_backbones:HierarchicalMMDiT",
        "ssm_dit": "dew_b200.models.diffusion_backbones:SSMDiT", "jepa_encoder": "dew_b200.models.diffusion_backbones:JepaEncoder",
        "jepa_video_encoder": "dew_b200.models.diffusion_backbones:JepaVideoEncoder",
        "flux": "dew_b200.models.latent_backbones:RectifiedFlowTransformer", "flux2": "dew_b200.models.latent_backbones:Flux2",
        "qwen_image": "dew_b200.models.latent_backbones:QwenImage", "z_image": "dew_b200.models.latent_backbones:ZImage",
        "sd3": "dew_b200.models.latent_backbones:SD3Transformer", "wan": "dew_b200.models.latent_backbones:WanTransformer",
        "edm2": "dew_b200.models.latent_backbones:EDM2UNet",
        "kl_vae": "dew_b200.models.autoencoders:KLAutoEncoder", "vit": "dew_b200.models.autoencoders:ViT",
        "autoencoder_kl": "dew_b200.models.latent_autoencoders:AutoencoderKL", "dc_ae": "dew_b200.models.latent_autoencoders:DCAE",
        "causal_video_vae": "dew_b200.models.latent_autoencoders:CausalVideoVAE",
        "classic_decoder": "dew_b200.models.classic_decoder:ClassicDecoder",
    },
    "objective": {
        "lm": "dew_b200.objectives.lm:LMObjective",
        "diffusion": "dew_b200.objectives.diffusion:DiffusionObjective",
        "jepa": "dew_b200.objectives.jepa:JEPAObjective",
        "supervised": "dew_b200.objectives.supervised:SupervisedObjective",
    },
    "optimizer": {"optim": "dew_b200.optim.config:OptimConfig"},
    "tokenizer": {"bytes": "dew_b200.data.tokenizer:ByteTokenizer"},
    "dataset": {"memory": "dew_b200.data.dataset:Memory", "token_files": "dew_b200.data.dataset:TokenFiles",
                "jsonl": "dew_b200.data.sources:JsonLines", "parquet": "dew_b200.data.sources:Parquet", "hub": "dew_b200.data.sources:Hub"},
}
_TRUSTED = {"dew_b200", "torch", "builtins"}


class Unrecordable(TypeError):
    """A value that no record can carry (a tensor, an open file, a lambda)."""


class Aliases(Mapping):
    """One kind's table of names: static entries (import paths, resolved on first read) and registered objects."""

    def __init__(self, kind: str):
        self.kind = kind
        self._paths: Dict[str, str] = dict(_STATIC.get(kind, {}))
        self._objects: Dict[str, Any] = {}

    def register(self, name: str) -> Callable[[Any], Any]:
        def deco(obj: Any) -> Any:
            held = self._objects.get(name)
            if held is not None and held is not obj:
                raise ValueError(f"{self.kind} {name!r} is already registered")
            static = self._paths.get(name)
            if static is not None and static != import_path(obj):
                raise ValueError(f"{self.kind} {name!r} already names {static}")
            self._objects[name] = obj
            return obj
        return deco

    def __getitem__(self, name: str) -> Any:
        if name in self._objects:
            return self._objects[name]
        if name in self._paths:
            obj = imported(self._paths[name])
            self._objects[name] = obj
            return obj
        raise KeyError(f"unknown {self.kind} {name!r}; known: {sorted(self)}")

    def __iter__(self) -> Iterator[str]:
        return iter(sorted(set(self._paths) | set(self._objects)))

    def __len__(self) -> int:
        return len(set(self._paths) | set(self._objects))

    def __contains__(self, name: object) -> bool:
        return name in self._paths or name in self._objects

    def __setitem__(self, name: str, obj: Any) -> None:       # the dict-style use older call sites make
        self.register(name)(obj)

    def path_of(self, name: str) -> str:
        return self._paths[name] if name in self._paths else import_path(self._objects[name])


_TABLES: Dict[str, Aliases] = {}


def registry(kind: str) -> Aliases:
    if kind not in _TABLES:
        _TABLES[kind] = Aliases(kind)
    return _TABLES[kind]


def register(name: str, kind: str = "model") -> Callable[[Any], Any]:
    return registry(kind).register(name)


def lookup(name: str, kind: str = "model") -> Any:
    return registry(kind)[name]


# ------------------------------------------------------------------------------------------------ import paths
def import_path(member: Any) -> str:
    """``module:QualName`` of a class or function defined at module level."""
    mod, qual = getattr(member, "__module__", None), getattr(member, "__qualname__", None)
    if not mod or not qual or "<locals>" in qual or "<lambda>" in qual:
        raise Unrecordable(f"{member!r} has no import path (define it at module level)")
    return f"{mod}:{qual}"


def trust_sources(names: Sequence[str]) -> None:
    """Let records import classes from these top-level packages (beside this package and torch)."""
    _TRUSTED.update(n.split(".")[0] for n in names)


def trusts_source(path: str) -> bool:
    return path.split(":")[0].split(".")[0] in _TRUSTED


def imported(path: str, trust: Sequence[str] = ()) -> Any:
    """The object at ``module:QualName``; the module's top-level package must be trusted (a record is data: it must not be
    able to import arbitrary code)."""
    if ":" not in path:
        raise ValueError(f"{path!r} is not an import path of the form 'package.module:Name'")
    if not trusts_source(path) and path.split(":")[0].split(".")[0] not in {t.split(".")[0] for t in trust}:
        raise PermissionError(f"{path!r} lies outside the trusted packages {sorted(_TRUSTED)}; call trust_sources([...]) to admit it")
    mod, qual = path.split(":", 1)
    obj: Any = importlib.import_module(mod)
    for part in qual.split("."):
        obj = getattr(obj, part)
    return obj


# ------------------------------------------------------------------------------------------------ writing records
def _constructor_fields(value: Any) -> Dict[str, Any]:
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        return {f.name: getattr(value, f.name) for f in dataclasses.fields(value) if f.init}
    kept = getattr(value, "__record_fields__", None)
    if kept is not None:
        return dict(kept() if callable(kept) else kept)
    sig = inspect.signature(type(value).__init__)
    out = {}
    for name, p in list(sig.parameters.items())[1:]:
        if p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
            continue
        if not hasattr(value, name):
            raise Unrecordable(f"{type(value).__name__} does not keep its constructor argument {name!r}: make it a dataclass, "
                               "keep the argument as an attribute, or define __record_fields__")
        out[name] = getattr(value, name)
    return out


def to_record(value: Any) -> Any:
    """JSON-able record of ``value``: scalars and strings as they are, sequences and mappings element-wise, enums by name,
    dtypes by name, functions and classes by import path, objects as ``{"class": path, "fields": {...}}``."""
    import torch
    if value is None or isinstance(value, (bool, int, float, str)):
        return value
    if isinstance(value, enum.Enum):
        return {"enum": import_path(type(value)), "name": value.name}
    if isinstance(value, torch.dtype):
        return {"dtype": str(value).replace("torch.", "")}
    if isinstance(value, torch.Tensor):
        raise Unrecordable("a tensor does not belong in a record: store it in a checkpoint item")
    if isinstance(value, (list, tuple)):
        return [to_record(v) for v in value]
    if isinstance(value, Mapping):
        return {str(k): to_record(v) for k, v in value.items()}
    if isinstance(value, type) or inspect.isfunction(value) or inspect.isbuiltin(value):
        return {"function": import_path(value)}
    return {"class": import_path(type(value)), "fields": {k: to_record(v) for k, v in _constructor_fields(value).items()}}


# ------------------------------------------------------------------------------------------------ reading records
def _convert(annotation: Any, value: Any, trust: Sequence[str]) -> Any:
    """``value`` (as JSON gave it) as the type ``annotation`` declares."""
    import torch
    if isinstance(value, Mapping) and ("class" in value or "function" in value or "enum" in value or "dtype" in value):
        return from_record(value, trust=trust)
    origin = typing.get_origin(annotation)
    args = typing.get_args(annotation)
    if origin in (Union, types.UnionType):
        for a in args:
            if a is type(None):
                if value is None:
                    return None
                continue
            try:
                return _convert(a, value, trust)
            except (TypeError, ValueError):
                continue
        return value
    if origin in (tuple, Tuple) or annotation is tuple:
        if isinstance(value, (list, tuple)):
            inner = args[0] if args and (len(args) == 2 and args[1] is Ellipsis) else None
            return tuple(_convert(inner, v, trust) if inner is not None else (_convert(args[i], v, trust) if i < len(args) else v) for i, v in enumerate(value))
        return value
    import collections.abc as cabc
    if origin in (cabc.Sequence, cabc.Collection, cabc.Iterable) and isinstance(value, (list, tuple)):
        return tuple(_convert(args[0] if args else Any, v, trust) for v in value)       # a declared sequence reads back immutable
    if origin in (list, typing.List) or annotation is list:
        return [_convert(args[0] if args else Any, v, trust) for v in value] if isinstance(value, (list, tuple)) else value
    if annotation is torch.dtype and isinstance(value, str):
        return getattr(torch, value)
    if annotation is float and isinstance(value, int) and not isinstance(value, bool):
        return float(value)
    if dataclasses.is_dataclass(annotation) and isinstance(value, Mapping):
        return _build(annotation, value, trust)
    if isinstance(value, list):
        return [_convert(Any, v, trust) for v in value]
    if isinstance(value, Mapping):
        return {k: _convert(Any, v, trust) for k, v in value.items()}
    return value


def _build(member: Any, fields: Mapping[str, Any], trust: Sequence[str]) -> Any:
    target = member.__init__ if isinstance(member, type) else member
    sig = inspect.signature(target)
    params = {n: p for n, p in sig.parameters.items() if n != "self"}
    takes_any = any(p.kind is p.VAR_KEYWORD for p in params.values())
    unknown = [k for k in fields if k not in params and not takes_any]
    if unknown:
        known = [n for n, p in params.items() if p.kind not in (p.VAR_POSITIONAL, p.VAR_KEYWORD)]
        raise TypeError(f"{getattr(member, '__name__', member)} has no field(s) {unknown}; its fields are {known}")
    try:
        hints = typing.get_type_hints(target)
    except Exception:
        hints = {}
    kwargs = {k: _convert(hints.get(k, Any), v, trust) for k, v in fields.items()}
    return member(**kwargs)


def from_record(record: Any, kind: Optional[str] = None, trust: Sequence[str] = ()) -> Any:
    """Rebuild what ``to_record`` wrote.  ``record["class"]`` may be an import path or, with ``kind``, an alias of that kind."""
    import torch
    if not isinstance(record, Mapping):
        return _convert(Any, record, trust)
    if "dtype" in record and len(record) == 1:
        return getattr(torch, record["dtype"])
    if "enum" in record:
        return imported(record["enum"], trust)[record["name"]]
    if "function" in record:
        name = record["function"]
        return imported(name, trust) if ":" in name else lookup(name, kind or "model")
    if "class" in record:
        name = record["class"]
        extra = set(record) - {"class", "fields"}
        if extra:
            raise TypeError(f"a record holds 'class' and 'fields' only, not {sorted(extra)}")
        member = imported(name, trust) if ":" in name else lookup(name, kind or "model")
        return _build(member, record.get("fields", {}), trust)
    return {k: from_record(v, None, trust) for k, v in record.items()}
