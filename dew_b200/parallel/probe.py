"""Measure what a job's collectives cost on this machine: link bandwidth per collective and message size (device-timed,
max over ranks) and the device memory a communicator takes.

``probe(group)`` times all-gather, reduce-scatter, all-reduce, all-to-all and a neighbour exchange at a few payload
sizes and returns a ``Link`` table (algorithmic and bus bandwidth in GB/s); parallel layouts read it to decide, for
instance, whether tensor-parallel activations are worth spreading (sequence-parallel) - the reference takes that decision
from the same kind of measurement.  ``communicator_memory`` reports the bytes the first collective of a fresh process
group allocates, measured around its creation.  On CPU ranks (gloo) the same code runs with wall-clock timing, which is
how it is tested.

Reference: src/dew/training/distributed.py:83-131 (``Link``, probe all-gather of 256 MiB), src/dew/communicators.py:624-630
(communicator memory measured in an isolated process), src/dew/nn/sharding.py:262-280 (``SPREAD`` decided by bandwidth).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass
class LinkRow:
    collective: str
    bytes: int
    ms: float
    algbw_gbs: float       # payload bytes / time
    busbw_gbs: float       # bytes that cross a rank's links / time (the figure comparable between collectives)


@dataclass
class Link:
    world: int
    rows: List[LinkRow] = field(default_factory=list)

    def best(self, collective: str) -> float:
        vals = [r.busbw_gbs for r in self.rows if r.collective == collective]
        return max(vals) if vals else 0.0

    def spread_pays(self, threshold_gbs: float = 283.0) -> bool:
        """Whether sequence-parallel (reduce-scatter + all-gather) tensor-parallel activations beat one all-reduce: they
        move the same bytes in two collectives, so they pay once the links are fast enough to hide the extra launch."""
        return min(self.best("reduce_scatter"), self.best("all_gather")) >= threshold_gbs

    def table(self) -> str:
        out = [f"{'collective':<15} {'MiB':>9} {'ms':>9} {'alg GB/s':>9} {'bus GB/s':>9}"]
        for r in self.rows:
            out.append(f"{r.collective:<15} {r.bytes / 2**20:>9.1f} {r.ms:>9.3f} {r.algbw_gbs:>9.1f} {r.busbw_gbs:>9.1f}")
        return "\n".join(out)


_BUS = {"all_reduce": lambda w: 2 * (w - 1) / w, "all_gather": lambda w: (w - 1) / w, "reduce_scatter": lambda w: (w - 1) / w,
        "all_to_all": lambda w: (w - 1) / w, "exchange": lambda w: 1.0}


def _time(fn, device, iters: int, group) -> float:
    fn()
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            fn()
        end.record()
        torch.cuda.synchronize(device)
        ms = start.elapsed_time(end) / iters
    else:
        dist.barrier(group=group)
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        ms = 1000 * (time.perf_counter() - t0) / iters
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def probe(group: Optional[dist.ProcessGroup] = None, sizes: Sequence[int] = (1 << 20, 1 << 24, 1 << 28), device=None, iters: int = 5,
          collectives: Sequence[str] = ("all_reduce", "all_gather", "reduce_scatter", "all_to_all", "exchange")) -> Link:
    """``sizes``: total payload bytes per rank of each measurement (bf16 elements)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    device = torch.device(device if device is not None else ("cuda" if dist.get_backend(group) == "nccl" else "cpu"))
    link = Link(world)
    for nbytes in sizes:
        n = max(world, nbytes // 2 // world * world)
        x = torch.ones(n, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32, device=device)
        shard = x[: n // world].clone()
        out = torch.empty_like(x)
        peer = (rank + 1) % world
        fns = {
            "all_reduce": lambda: dist.all_reduce(x, group=group),
            "all_gather": lambda: dist.all_gather_into_tensor(out, shard, group=group) if device.type == "cuda"
            else dist.all_gather(list(out.chunk(world)), shard, group=group),
            "reduce_scatter": lambda: dist.reduce_scatter_tensor(shard, x, group=group) if device.type == "cuda"
            else dist.all_reduce(x, group=group),
            "all_to_all": lambda: dist.all_to_all_single(out, x, group=group) if device.type == "cuda"
            else dist.all_gather(list(out.chunk(world)), shard, group=group),
            "exchange": lambda: [w.wait() for w in dist.batch_isend_irecv(
                [dist.P2POp(dist.isend, shard, peer, group), dist.P2POp(dist.irecv, out[: n // world], (rank - 1) % world, group)])],
        }
        payload = x.numel() * x.element_size()
        for name in collectives:
            if world == 1 and name == "exchange":
                continue
            ms = _time(fns[name], device, iters, group)
            size = payload if name != "exchange" else payload // world
            alg = size / ms / 1e6
            link.rows.append(LinkRow(name, size, ms, alg, alg * _BUS[name](world)))
    return link


def communicator_memory(device=None) -> Dict[str, int]:
    """Device bytes taken by creating a fresh process group and running its first collective (0 on CPU ranks)."""
    device = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() and dist.get_backend() == "nccl" else "cpu"))
    if device.type != "cuda":
        g = dist.new_group(list(range(dist.get_world_size())))
        dist.all_reduce(torch.ones(1), group=g)
        return {"bytes": 0}
    torch.cuda.synchronize(device)
    free0, _ = torch.cuda.mem_get_info(device)
    g = dist.new_group(list(range(dist.get_world_size())))
    dist.all_reduce(torch.ones(1, device=device), group=g)
    torch.cuda.synchronize(device)
    free1, _ = torch.cuda.mem_get_info(device)
    return {"bytes": max(0, free0 - free1)}
