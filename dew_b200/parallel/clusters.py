"""Cluster environments: how a process learns the coordinator address, the process count and its rank.

Parity: src/dew/clusters.py (``Joining`` :54, ``ClusterEnvironment`` :69, ``OpenMPI`` :138, ``Slurm`` :170,
``Kubernetes`` :252, ``detected_environment`` :283) plus torchrun's own variables.  A custom scheduler is any class
with ``name``, ``detected()`` and ``joining() -> Joining``.
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass
from typing import List, Mapping, Optional, Type


@dataclass(frozen=True)
class Joining:
    coordinator: str          # host:port
    count: int
    rank: int
    local_rank: int = 0
    detection: str = ""


class ClusterEnvironment:
    name = "base"

    def __init__(self, env: Optional[Mapping[str, str]] = None):
        self.env = dict(os.environ if env is None else env)

    def detected(self) -> bool:
        raise NotImplementedError

    def joining(self) -> Joining:
        raise NotImplementedError


class TorchRun(ClusterEnvironment):
    name = "torchrun"

    def detected(self):
        return all(k in self.env for k in ("RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"))

    def joining(self):
        e = self.env
        return Joining(f"{e['MASTER_ADDR']}:{e['MASTER_PORT']}", int(e["WORLD_SIZE"]), int(e["RANK"]), int(e.get("LOCAL_RANK", 0)), self.name)


class OpenMPI(ClusterEnvironment):
    name = "openmpi"

    def detected(self):
        return "OMPI_COMM_WORLD_SIZE" in self.env

    def joining(self):
        e = self.env
        host = e.get("DEWB_COORDINATOR") or e.get("MASTER_ADDR", "127.0.0.1")
        port = e.get("MASTER_PORT", "29400")
        return Joining(f"{host}:{port}", int(e["OMPI_COMM_WORLD_SIZE"]), int(e["OMPI_COMM_WORLD_RANK"]),
                       int(e.get("OMPI_COMM_WORLD_LOCAL_RANK", 0)), self.name)


def _first_slurm_host(nodelist: str) -> str:
    """``node[03-05,09]`` -> ``node03``; ``a,b`` -> ``a``."""
    m = re.match(r"([^\[,]+)\[([^\]]+)\]", nodelist)
    if not m:
        return nodelist.split(",")[0]
    first = m.group(2).split(",")[0].split("-")[0]
    return m.group(1) + first


class Slurm(ClusterEnvironment):
    name = "slurm"

    def detected(self):
        return "SLURM_PROCID" in self.env and "SLURM_NTASKS" in self.env

    def joining(self):
        e = self.env
        host = _first_slurm_host(e.get("SLURM_STEP_NODELIST") or e.get("SLURM_JOB_NODELIST", "127.0.0.1"))
        port = e.get("MASTER_PORT") or str(29400 + int(e.get("SLURM_JOB_ID", "0")) % 1000)
        return Joining(f"{host}:{port}", int(e["SLURM_NTASKS"]), int(e["SLURM_PROCID"]), int(e.get("SLURM_LOCALID", 0)), self.name)


class Kubernetes(ClusterEnvironment):
    """Indexed Jobs / StatefulSets: ``JOB_COMPLETION_INDEX`` or the pod name's ordinal is the rank."""
    name = "kubernetes"

    def detected(self):
        return "KUBERNETES_SERVICE_HOST" in self.env and ("JOB_COMPLETION_INDEX" in self.env or "DEWB_REPLICAS" in self.env)

    def joining(self):
        e = self.env
        rank = int(e.get("JOB_COMPLETION_INDEX", re.sub(r".*-", "", e.get("HOSTNAME", "0")) or 0))
        return Joining(f"{e.get('DEWB_COORDINATOR', 'localhost')}:{e.get('MASTER_PORT', '29400')}", int(e.get("DEWB_REPLICAS", 1)), rank, 0, self.name)


ENVIRONMENTS: List[Type[ClusterEnvironment]] = [TorchRun, OpenMPI, Slurm, Kubernetes]


def detected_environment(env: Optional[Mapping[str, str]] = None, extra: Optional[List[Type[ClusterEnvironment]]] = None) -> Optional[ClusterEnvironment]:
    for cls in list(extra or []) + ENVIRONMENTS:
        c = cls(env)
        if c.detected():
            return c
    return None
