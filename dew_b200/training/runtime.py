"""Process start-up: join the pool, pick the device, install failure handling and the preemption handler.

Parity: src/dew/training/runtime.py (``prepare_process`` :76-120, ``_join_process_pool`` :239-274, ``Preempted`` /
``PreemptionNotice`` :305-465).
"""
from __future__ import annotations

import datetime
import os
import signal
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..parallel.clusters import ClusterEnvironment, Joining, detected_environment
from ..parallel.coordination import Pool, end_pool_on_failure


@dataclass
class ProcessContext:
    joining: Optional[Joining]
    pool: Optional[Pool]
    device: torch.device


class PreemptionNotice:
    """SIGTERM sets ``requested``; the trainer checkpoints at the next agreed step and exits 143."""

    def __init__(self):
        self.requested = False

    def install(self):
        def handler(signum, frame):
            self.requested = True
        try:
            signal.signal(signal.SIGTERM, handler)
        except ValueError:
            pass
        return self


def prepare_process(multi_host: Optional[bool] = None, cluster: Optional[ClusterEnvironment] = None, backend: Optional[str] = None,
                    timeout_s: float = 1800.0, failure_watch: bool = True) -> ProcessContext:
    """Join the process pool named by the environment (torchrun / Open MPI / Slurm / Kubernetes), select this rank's GPU
    and start the failure watcher. With no cluster environment the process runs alone."""
    env = cluster or detected_environment()
    cuda = torch.cuda.is_available()
    if env is None or (multi_host is False):
        return ProcessContext(None, None, torch.device("cuda", 0) if cuda else torch.device("cpu"))
    j = env.joining()
    host, port = j.coordinator.rsplit(":", 1)
    os.environ.setdefault("MASTER_ADDR", host)
    os.environ.setdefault("MASTER_PORT", port)
    os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
    device = torch.device("cuda", j.local_rank) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    if not dist.is_initialized():
        dist.init_process_group(backend or ("nccl" if cuda else "gloo"), rank=j.rank, world_size=j.count,
                                timeout=datetime.timedelta(seconds=timeout_s), **({"device_id": device} if cuda else {}))
    pool = None
    try:
        store = dist.distributed_c10d._get_default_store()
        pool = Pool(store, j.rank, j.count)
        if failure_watch:
            end_pool_on_failure(pool)
    except Exception:
        pool = None
    return ProcessContext(j, pool, device)
