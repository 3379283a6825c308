"""``Checkpoints``: a run directory of step sub-directories, each a composite of the items ``model`` / ``resume`` /
``profiles``, beside ``run.json`` and the ``frozen/<digest>`` store.

On-disk structure (the reference's: src/dew/checkpoints/__init__.py:1-60,150-180; _payloads.py:1-172)::

    <directory>/run.json                         how to rebuild the task (model / objective / tokenizer record)
    <directory>/frozen/<digest>/                 every non-``params`` variables collection, stored once by content
    <directory>/<step>/model/                    step, microstep, updates, variables, ema (EMA as XOR byte planes)
    <directory>/<step>/resume/                   opt_state, key, scale, accumulation, consumed, data position
    <directory>/<step>/profiles/                 post-hoc EMA power-profile averages
    <directory>/<step>/projected.json            which items retention kept for this step
    <directory>/<step>/metadata.json             metrics, ranking, rung, artifact, encoded EMA leaves, frozen digests

Inside an item the tree is stored as ``tree.safetensors`` keyed by the same tree paths the reference's PyTree has
(``variables/params/<module path>/kernel`` ...) plus ``_METADATA.json`` (paths, shapes, dtypes).  An ``orbax`` codec
is used instead when ``orbax-checkpoint`` is importable and requested.  Saving is asynchronous (``wait()`` joins);
restore places leaves on whatever device / sharding the template has.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import threading
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Union

import torch

from ..training.state import MODEL_STATE, TrainState
from ..utils.files import atomic_write_json, read_json
from ..utils.trees import flatten, unflatten
from . import state_trees as ST
from . import tensors as TS

RUN_FILE = "run.json"
FROZEN_STORE = "frozen"
ROLES = ("model", "profiles", "resume")
ONE_ITEM = "default"
PROJECTED = "projected.json"
METADATA = "metadata.json"
_NEEDS = {"model": ("model",), "resume": ROLES}


class NonFiniteState(RuntimeError):
    pass


@dataclass(frozen=True)
class Keep:
    """Retention: ``Keep.latest`` keeps one step, ``Keep(n)`` the newest n, ``Keep.all`` everything; ``every`` also
    keeps each multiple of it; ``model_only_older`` cuts older kept steps down to their ``model`` item."""
    count: Optional[int] = 1
    every: Optional[int] = None
    model_only_older: bool = False


Keep.latest = Keep(1)
Keep.all = Keep(None)


@dataclass(frozen=True)
class Ranking:
    """Keep the best ``count`` steps by ``metric`` (``mode`` 'min' or 'max') besides what ``Keep`` keeps."""
    metric: str
    mode: str = "min"
    count: int = 1

    def better(self, a: float, b: float) -> bool:
        return a < b if self.mode == "min" else a > b


def _digest_tree(flat: Mapping[str, torch.Tensor]) -> str:
    h = hashlib.sha256()
    for k in sorted(flat):
        t = flat[k]
        h.update(k.encode())
        if isinstance(t, torch.Tensor):
            h.update(str(t.dtype).encode())
            h.update(str(tuple(t.shape)).encode())
            h.update(TS._bytes(t))
    return h.hexdigest()[:32]


def _to_cpu(flat: Mapping[str, Any]) -> Dict[str, Any]:
    out = {}
    for k, v in flat.items():
        if isinstance(v, torch.Tensor):
            full = v.full_tensor() if hasattr(v, "full_tensor") else v
            out[k] = full.detach().to("cpu", copy=True)
        else:
            out[k] = v
    return out


def _split_scalars(flat: Mapping[str, Any]):
    tensors, scalars = {}, {}
    for k, v in flat.items():
        if isinstance(v, torch.Tensor):
            tensors[k] = v
        elif v is not None:
            scalars[k] = v
    return tensors, scalars


class CorruptCheckpoint(RuntimeError):
    """A step whose files do not match the digests written with them."""


def _file_sha256(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 22), b""):
            h.update(block)
    return h.hexdigest()


class Checkpoints:
    def __init__(self, directory: os.PathLike, *, keep: Union[Keep, int] = Keep.latest,
                 local_directory: Optional[os.PathLike] = None, local_every: Optional[int] = None,
                 ranking: Optional[Ranking] = None, kinds: Optional[Mapping[str, str]] = None,
                 process_index: int = 0, process_count: int = 1, verify_on_read: bool = True):
        self.directory = Path(directory)
        self.verify_on_read = verify_on_read        # check every item's file digest when it is read
        self.keep = Keep(keep) if isinstance(keep, int) else keep
        self.local_directory = Path(local_directory) if local_directory else None
        self.local_every = local_every
        self.ranking = ranking
        self.kinds = dict(kinds) if kinds else None
        self.process_index, self.process_count = process_index, process_count
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None

    # ------------------------------------------------------------------ listing
    def steps(self) -> List[int]:
        if not self.directory.exists():
            return []
        out = []
        for p in self.directory.iterdir():
            if p.is_dir() and p.name.isdigit() and (p / METADATA).exists():
                out.append(int(p.name))
        return sorted(out)

    def latest(self) -> Optional[int]:
        s = self.steps()
        return s[-1] if s else None

    def best(self) -> Optional[int]:
        if self.ranking is None:
            return None
        scored = []
        for s in self.steps():
            m = read_json(self.directory / str(s) / METADATA).get("metrics", {})
            if self.ranking.metric in m:
                scored.append((m[self.ranking.metric], s))
        if not scored:
            return None
        return (min(scored) if self.ranking.mode == "min" else max(scored))[1]

    def metadata(self, step: Optional[int] = None) -> Dict[str, Any]:
        step = self.latest() if step is None else step
        return read_json(self.directory / str(step) / METADATA)

    def verify(self, step: Optional[int] = None) -> Dict[str, bool]:
        """Per item of ``step``: whether its tensor file still has the digest recorded when it was written (items written
        before digests were recorded count as intact)."""
        step = self.latest() if step is None else step
        out = {}
        root = self.directory / str(step)
        for d in sorted(p for p in root.iterdir() if p.is_dir()):
            meta, data = d / "_METADATA.json", d / "tree.safetensors"
            if not meta.exists():
                continue
            want = read_json(meta).get("sha256")
            out[d.name] = data.exists() and (want is None or _file_sha256(data) == want)
        return out

    def resumed(self, resume: str = "auto") -> Optional[int]:
        """The step a run resumes from under ``resume`` = 'auto' | 'require' | 'never': the newest step whose files are
        intact (a step cut short or damaged on disk is passed over for the one before it, with a warning)."""
        if resume == "never":
            return None
        for step in reversed(self.steps()):
            try:
                intact = all(self.verify(step).values())
            except OSError:
                intact = False
            if intact:
                return step
            import warnings
            warnings.warn(f"checkpoint step {step} in {self.directory} failed its integrity check; trying the step before it")
        if resume == "require":
            raise FileNotFoundError(f"resume='require' but {self.directory} holds no intact checkpoint")
        return None

    # ------------------------------------------------------------------ run record
    def write_run(self, record: Mapping[str, Any]) -> None:
        if self.process_index == 0:
            atomic_write_json(self.directory / RUN_FILE, dict(record))

    def read_run(self) -> Optional[Dict[str, Any]]:
        p = self.directory / RUN_FILE
        return read_json(p) if p.exists() else None

    # ------------------------------------------------------------------ save
    def _write_item(self, root: Path, item: str, flat: Mapping[str, Any]) -> None:
        d = root / item
        d.mkdir(parents=True, exist_ok=True)
        tensors, scalars = _split_scalars(flat)
        TS.save_file(tensors, d / "tree.safetensors")
        atomic_write_json(d / "_METADATA.json", {
            "tree": {k: {"shape": list(v.shape), "dtype": str(v.dtype)} for k, v in tensors.items()},
            "scalars": scalars, "sha256": _file_sha256(d / "tree.safetensors")})

    def save(self, step: int, state: Union[TrainState, Mapping[str, Any]], saved: Optional[Mapping[str, Any]] = None,
             metrics: Optional[Mapping[str, float]] = None, *, weights_only: bool = False, rung: Any = None,
             artifact: Any = None, training: Any = None, tokenizer: Any = None, blocking: bool = False) -> None:
        """Snapshot ``state`` (copied to host now) and write it in the background.  ``saved`` carries the data
        position; ``metrics`` feed ranking / ``best()``."""
        self.wait()
        if not isinstance(state, TrainState):
            payload = {ONE_ITEM: _to_cpu(flatten(state))}
            meta = {"kind": "mapping"}
        else:
            weights = ST.to_stored(state.variables.get("params", {}), self.kinds)
            for t in weights.values():
                if isinstance(t, torch.Tensor) and t.dtype.is_floating_point and not bool(torch.isfinite(t.float()).all()):
                    raise NonFiniteState(f"refusing to save step {step}: a parameter is not finite")
            model: Dict[str, Any] = {"step": state.step, "microstep": state.microstep, "updates": state.updates}
            model.update({f"variables/params/{k}": v for k, v in weights.items()})
            frozen_digests = {}
            for coll, tree in state.variables.items():
                if coll == "params":
                    continue
                flat = _to_cpu(flatten(tree))
                digest = _digest_tree(flat)
                frozen_digests[coll] = digest
                froot = self.directory / FROZEN_STORE / digest
                if self.process_index == 0 and not froot.exists():
                    self._write_item(self.directory / FROZEN_STORE, digest, flat)
            encoded: List[str] = []
            if state.ema is not None:
                ema_w = ST.to_stored(state.ema.get("params", {}), self.kinds)
                cpu_w, cpu_e = _to_cpu(weights), _to_cpu(ema_w)
                planes, encoded = ST.encode_ema(cpu_e, cpu_w)
                model.update({f"ema/params/{k}": v for k, v in planes.items()})
            payload = {"model": _to_cpu(model)}
            if not weights_only:
                resume: Dict[str, Any] = {"key": int(state.key)}
                # every tree of the optimizer state that mirrors the parameters (mu / nu, M3's slow / chunk / slow_direction,
                # any later optimizer's) is stored leaf by leaf under the parameters' stored names; the rest (count, ...)
                # as tensors or plain scalars
                for k, v in state.opt_state.items():
                    if k == "profiles":
                        continue
                    if isinstance(v, Mapping):
                        st = ST.to_stored(v, self.kinds)
                        resume.update({f"opt_state/{k}/params/{kk}": vv for kk, vv in st.items()})
                    else:
                        resume[f"opt_state/{k}"] = v
                if state.scale is not None:
                    resume.update({f"scale/{k}": v for k, v in flatten(state.scale).items()})
                resume.update({f"consumed/{k}": int(v) for k, v in state.consumed.items()})
                if saved:
                    resume.update({f"data/{k}": v for k, v in flatten(dict(saved)).items()})
                payload["resume"] = _to_cpu(resume)
                profiles = state.opt_state.get("profiles") if isinstance(state.opt_state, Mapping) else None
                if profiles:
                    payload["profiles"] = _to_cpu({f"averages/{k}": v for k, v in flatten(profiles).items()})
                    payload["resume"] = {k: v for k, v in payload["resume"].items() if not k.startswith("opt_state/profiles")}
            meta = {"kind": "train_state", "ema_planes": encoded, "frozen": frozen_digests}
        meta.update({"step": int(step), "metrics": {k: float(v) for k, v in (metrics or {}).items()},
                     "rung": rung, "artifact": artifact, "training": training, "items": sorted(payload)})

        def write():
            try:
                if self.process_index != 0:
                    return
                root = self.directory / str(int(step))
                tmp = self.directory / f".{int(step)}.partial"
                if tmp.exists():
                    shutil.rmtree(tmp)
                tmp.mkdir(parents=True)
                for item, flat in payload.items():
                    self._write_item(tmp, item, flat)
                atomic_write_json(tmp / PROJECTED, {"items": sorted(payload)})
                atomic_write_json(tmp / METADATA, meta)     # written last: its presence marks a complete step
                if root.exists():
                    shutil.rmtree(root)
                os.replace(tmp, root)
                self._retain()
            except BaseException as e:  # surfaced by wait()
                self._error = e

        if blocking:
            write()
            self._raise()
        else:
            self._thread = threading.Thread(target=write, name=f"checkpoint-{step}", daemon=True)
            self._thread.start()

    def save_local(self, step: int, state: TrainState) -> None:
        """Emergency checkpoint: every process writes what it holds under ``local_directory/<process>``."""
        if self.local_directory is None:
            return
        local = Checkpoints(self.local_directory / str(self.process_index), keep=Keep(1), kinds=self.kinds)
        local.save(step, state, blocking=True)

    def _raise(self):
        if self._error is not None:
            e, self._error = self._error, None
            raise e

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        self._raise()

    def close(self) -> None:
        self.wait()

    def _retain(self) -> None:
        steps = self.steps()
        keep = set()
        if self.keep.count is None:
            keep.update(steps)
        else:
            keep.update(steps[-self.keep.count:])
        if self.keep.every:
            keep.update(s for s in steps if s % self.keep.every == 0)
        if self.ranking is not None:
            scored = []
            for s in steps:
                m = read_json(self.directory / str(s) / METADATA).get("metrics", {})
                if self.ranking.metric in m:
                    scored.append((m[self.ranking.metric], s))
            scored.sort(reverse=self.ranking.mode == "max")
            keep.update(s for _, s in scored[: self.ranking.count])
        for s in steps:
            if s not in keep:
                shutil.rmtree(self.directory / str(s), ignore_errors=True)
            elif self.keep.model_only_older and s != steps[-1]:
                for item in ("resume", "profiles"):
                    shutil.rmtree(self.directory / str(s) / item, ignore_errors=True)
                atomic_write_json(self.directory / str(s) / PROJECTED, {"items": ["model"]})

    # ------------------------------------------------------------------ restore
    def _read_item(self, step: int, item: str) -> Dict[str, Any]:
        d = self.directory / str(step) / item
        if not d.exists():
            raise FileNotFoundError(f"step {step} holds no {item!r} item (it may have been cut to its model item)")
        if self.verify_on_read:
            want = read_json(d / "_METADATA.json").get("sha256")
            if want is not None and _file_sha256(d / "tree.safetensors") != want:
                raise CorruptCheckpoint(f"{d / 'tree.safetensors'} does not match the digest written with it")
        out: Dict[str, Any] = dict(TS.load_file(d / "tree.safetensors"))
        out.update(read_json(d / "_METADATA.json").get("scalars", {}))
        return out

    def variables(self, step: Optional[int] = None, ema: Optional[bool] = None, template: Optional[Mapping[str, Any]] = None,
                  param_dtype: Optional[torch.dtype] = None, device="cpu") -> Dict[str, Any]:
        """The weights of a step (EMA if ``ema`` and one is stored) - the model item alone serves this."""
        self.wait()
        step = self.latest() if step is None else step
        if step is None:
            raise FileNotFoundError(f"{self.directory} holds no checkpoint")
        model = self._read_item(step, "model")
        meta = self.metadata(step)
        weights = {k[len("variables/params/"):]: v for k, v in model.items() if k.startswith("variables/params/")}
        has_ema = any(k.startswith("ema/params/") for k in model)
        use = weights
        if (ema or (ema is None and has_ema)) and has_ema:
            planes = {k[len("ema/params/"):]: v for k, v in model.items() if k.startswith("ema/params/")}
            use = ST.decode_ema(planes, weights, meta.get("ema_planes", []))
        if template is not None:
            paths = list(flatten(template.get("params", template)).keys())
            flat = ST.from_stored(use, self.kinds, paths)
        elif self.kinds:
            flat = ST.from_stored(use, self.kinds, list(self.kinds.keys()))
        else:
            flat = dict(use)
        cast = lambda t: t.to(device=device, dtype=param_dtype if (param_dtype and t.dtype.is_floating_point) else t.dtype)
        out = {"params": unflatten({k: cast(v) for k, v in flat.items()})}
        for coll, digest in meta.get("frozen", {}).items():
            d = self.directory / FROZEN_STORE / digest
            out[coll] = unflatten({k: v.to(device) for k, v in TS.load_file(d / "tree.safetensors").items()})
        return out

    def restore(self, template: Optional[TrainState] = None, step: Optional[int] = None) -> TrainState:
        """Rebuild a ``TrainState``.  With a ``template`` the restored leaves are copied *into* the template's
        tensors (keeping their device, dtype and sharding); without one a fresh host state is returned."""
        self.wait()
        step = self.latest() if step is None else step
        if step is None:
            raise FileNotFoundError(f"{self.directory} holds no checkpoint")
        meta = self.metadata(step)
        if meta.get("kind") == "mapping":
            return unflatten(self._read_item(step, ONE_ITEM))
        model = self._read_item(step, "model")
        weights_st = {k[len("variables/params/"):]: v for k, v in model.items() if k.startswith("variables/params/")}
        paths = list(flatten(template.variables["params"]).keys()) if template is not None else \
            (list(self.kinds.keys()) if self.kinds else list(weights_st.keys()))
        conv = (lambda st: ST.from_stored(st, self.kinds, paths)) if (self.kinds or template is not None) else dict
        params = conv(weights_st)
        ema = None
        if any(k.startswith("ema/params/") for k in model):
            planes = {k[len("ema/params/"):]: v for k, v in model.items() if k.startswith("ema/params/")}
            ema = {"params": unflatten(conv(ST.decode_ema(planes, weights_st, meta.get("ema_planes", []))))}
        state = TrainState(step=int(model["step"]), microstep=int(model["microstep"]), updates=int(model["updates"]),
                           variables={"params": unflatten(params)}, ema=ema)
        for coll, digest in meta.get("frozen", {}).items():
            d = self.directory / FROZEN_STORE / digest
            state.variables[coll] = unflatten(dict(TS.load_file(d / "tree.safetensors")))
        if "resume" in meta.get("items", []) and (self.directory / str(step) / "resume").exists():
            res = self._read_item(step, "resume")
            state.key = int(res.get("key", 0))
            opt: Dict[str, Any] = {}
            trees: Dict[str, Dict[str, Any]] = {}
            for k, v in res.items():
                if not k.startswith("opt_state/"):
                    continue
                name, _, rest = k[len("opt_state/"):].partition("/")
                if rest.startswith("params/"):
                    trees.setdefault(name, {})[rest[len("params/"):]] = v
                elif not rest:
                    opt[name] = v
            for name, st in trees.items():
                # a tree that mirrors the parameters converts back through their stored names; a narrower one (a state
                # kept for some leaves only) keeps the leaves it has
                try:
                    got = conv(st)
                except KeyError:
                    got = dict(st)
                opt[name] = unflatten(got)
            state.opt_state = opt
            state.consumed = {k[len("consumed/"):]: int(v) for k, v in res.items() if k.startswith("consumed/")}
            sc = {k[len("scale/"):]: v for k, v in res.items() if k.startswith("scale/")}
            state.scale = unflatten(sc) if sc else None
            data = {k[len("data/"):]: v for k, v in res.items() if k.startswith("data/")}
            state.deferred = unflatten(data) if data else None
        if template is not None:
            _copy_into(template.variables, state.variables)
            state.variables = template.variables
            if template.ema is not None and state.ema is not None:
                _copy_into(template.ema, state.ema)
                state.ema = template.ema
            if template.opt_state and state.opt_state:
                for name, tree in template.opt_state.items():
                    if isinstance(tree, Mapping) and isinstance(state.opt_state.get(name), Mapping):
                        _copy_into(tree, state.opt_state[name])
                        state.opt_state[name] = tree
        return state

    def posthoc_ema(self, std: float, step: Optional[int] = None) -> Dict[str, Any]:
        """Post-hoc EMA of relative width ``std`` from the stored power-profile averages (Karras et al. 2024)."""
        from ..optim.averaging import coefficients, gamma_of_std, posthoc_average
        steps, gammas, snaps = [], [], []
        for s in self.steps():
            d = self.directory / str(s) / "profiles"
            if not d.exists():
                continue
            flat = self._read_item(s, "profiles")
            by_gamma: Dict[str, Dict[str, Any]] = {}
            for k, v in flat.items():
                _, g, rest = k.split("/", 2)
                by_gamma.setdefault(g, {})[rest] = v
            for g, tree in by_gamma.items():
                steps.append(s); gammas.append(float(g)); snaps.append(tree)
        if not snaps:
            raise FileNotFoundError("no stored EMA profiles to reconstruct from")
        target = step if step is not None else max(steps)
        w = coefficients(steps, gammas, target, gamma_of_std(std))
        return unflatten(posthoc_average(snaps, w))


def _copy_into(dst_tree: Mapping[str, Any], src_tree: Mapping[str, Any]) -> None:
    dst, src = flatten(dst_tree), flatten(src_tree)
    with torch.no_grad():
        for k, d in dst.items():
            if k in src and isinstance(d, torch.Tensor):
                d.copy_(src[k].to(d.device, d.dtype))


__all__ = ["Checkpoints", "Keep", "Ranking", "NonFiniteState", "RUN_FILE", "FROZEN_STORE", "ROLES"]
