"""Local (per-process) checkpoints of sharded state, and recovery of a step one process lost from the processes that hold
the same shards.

Under hybrid sharding (``MeshSpec(fsdp=F, replicas=R)``) every shard of the masters / moments / EMA exists R times: on the
ranks that differ only along the replica axis.  ``save_local`` lets every rank write what it holds (fast, no gather, the
"emergency" checkpoint of the reference); when a rank comes back without its file (a replaced node, a wiped scratch
disk), ``restore_local`` finds for every lost shard a rank that still has it, which sends it over, and every rank ends
with the state of that step.  A shard no surviving rank holds makes the step unrecoverable, and the call says which.

Reference: src/dew/checkpoints/_replicas.py (``Grid``, ``_sources``, ``_covered``, ``_from_replicas``), local / emergency
checkpoints of src/dew/checkpoints/__init__.py (``local_directory``, ``local_every``).
"""
from __future__ import annotations

import json
import os
import shutil
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Mapping, Optional, Sequence

import torch
import torch.distributed as dist

from . import tensors as TS


@dataclass(frozen=True)
class ShardGrid:
    """Which ranks hold the same shards: ``holders[r]`` lists the ranks (``r`` included) that differ from ``r`` along the
    replica axes only."""
    world: int
    holders: Mapping[int, Sequence[int]]

    @classmethod
    def of(cls, mesh, replica_axes: Sequence[str]) -> "ShardGrid":
        return cls(mesh.world, {r: tuple(mesh.axis_ranks(tuple(replica_axes), r)) if replica_axes else (r,) for r in range(mesh.world)})

    def sources(self, have: Sequence[bool]) -> Dict[int, int]:
        """For every rank that lost its file, the rank to read its shards from; raises where no holder survives."""
        plan, missing = {}, []
        for r in range(self.world):
            if have[r]:
                continue
            alive = [h for h in self.holders[r] if have[h]]
            if not alive:
                missing.append(r)
            else:
                plan[r] = alive[(r // max(1, len(alive))) % len(alive)]        # spread the senders
        if missing:
            raise FileNotFoundError(f"the shards of rank(s) {missing} survive on no replica (holders: "
                                    f"{ {r: list(self.holders[r]) for r in missing} })")
        return plan


def _path(directory: os.PathLike, rank: int, step: int) -> Path:
    return Path(directory) / str(rank) / str(step)


def save_local(engine, state, step: int, directory: os.PathLike, keep: int = 1) -> Path:
    """This rank's shards (fp32 masters, moments, EMA) and the run's counters, written under ``<directory>/<rank>/<step>``;
    older local steps beyond ``keep`` are removed.  No collective."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    out = _path(directory, rank, step)
    tmp = out.with_name(out.name + ".partial")
    if tmp.exists():
        shutil.rmtree(tmp)
    tmp.mkdir(parents=True)
    tensors = {"master": engine.master, "m": engine.m, "v": engine.v}
    if engine.ema is not None:
        tensors["ema"] = engine.ema
    TS.save_file({k: t.detach().cpu() for k, t in tensors.items()}, tmp / "shards.safetensors")
    meta = {"step": int(state.step), "microstep": int(state.microstep), "updates": int(state.updates), "key": int(state.key),
            "count": int(state.opt_state["count"]), "consumed": dict(state.consumed), "shard_total": int(engine.shard_total),
            "rank": rank}
    (tmp / "meta.json").write_text(json.dumps(meta))
    if out.exists():
        shutil.rmtree(out)
    os.replace(tmp, out)
    steps = sorted(int(p.name) for p in out.parent.iterdir() if p.name.isdigit())
    for s in steps[:-keep] if keep else []:
        shutil.rmtree(out.parent / str(s), ignore_errors=True)
    return out


def restore_local(engine, state, step: int, directory: os.PathLike, grid: ShardGrid, group=None):
    """Collective.  Every rank loads its local file of ``step``; ranks without one receive their shards from a replica that
    has them.  Returns ``state`` with the step's counters; the compute copy is rebuilt from the restored masters."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    mine = _path(directory, rank, step)
    ok = (mine / "meta.json").exists() and (mine / "shards.safetensors").exists()
    have = [ok]
    if world > 1:
        flags = [None] * world
        dist.all_gather_object(flags, ok, group=group)
        have = [bool(f) for f in flags]
    plan = grid.sources(have)
    names = ["master", "m", "v"] + (["ema"] if engine.ema is not None else [])
    dest = {"master": engine.master, "m": engine.m, "v": engine.v, "ema": engine.ema}
    loaded, meta = None, None
    if ok:
        loaded = TS.load_file(mine / "shards.safetensors")
        meta = json.loads((mine / "meta.json").read_text())
    # holders send to the ranks they cover (same shard layout by construction); tensors travel through the CPU on gloo and
    # stay on the device on NCCL
    for lost, src in sorted(plan.items()):
        if rank == src:
            for n in names:
                dist.send(loaded[n].to(dest[n].device).contiguous(), dst=lost, group=group)
            dist.send(torch.tensor([meta[k] for k in ("step", "microstep", "updates", "key", "count")] +
                                   [meta["consumed"].get("examples", 0), meta["consumed"].get("tokens", 0)], dtype=torch.int64,
                                   device=dest["master"].device), dst=lost, group=group)
        elif rank == lost:
            loaded = {}
            for n in names:
                buf = torch.empty_like(dest[n])
                dist.recv(buf, src=src, group=group)
                loaded[n] = buf
            c = torch.empty(7, dtype=torch.int64, device=dest["master"].device)
            dist.recv(c, src=src, group=group)
            c = c.tolist()
            meta = {"step": c[0], "microstep": c[1], "updates": c[2], "key": c[3], "count": c[4], "consumed": {"examples": c[5], "tokens": c[6]}}
    with torch.no_grad():
        for n in names:
            dest[n].copy_(loaded[n].to(dest[n].device))
    engine.refresh_compute_copy()
    state.step, state.microstep, state.updates, state.key = meta["step"], meta["microstep"], meta["updates"], meta["key"]
    state.opt_state["count"] = torch.tensor(meta["count"], dtype=torch.int64)
    state.consumed = dict(meta["consumed"])
    return state


def local_steps(directory: os.PathLike, rank: int) -> List[int]:
    root = Path(directory) / str(rank)
    if not root.exists():
        return []
    return sorted(int(p.name) for p in root.iterdir() if p.name.isdigit() and (p / "meta.json").exists())
