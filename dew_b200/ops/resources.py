"""Launch / resource model: what each compiled kernel costs an SM and how many of its CTAs fit there.

Reads the ptxas report of the last build (registers per thread, spills, static shared memory) and combines it with the
launch shape a kernel is started with (threads per CTA, dynamic shared memory, tensor-memory columns) into the number of
co-resident CTAs per SM on sm_100a: 64 K registers, 227 KB shared memory (+1 KB reserved per CTA), 512 tensor-memory
columns, 2048 threads and 32 CTAs per SM.  The tests gate on it (a kernel that was designed for two CTAs per SM and
silently drops to one shows up here, on the CPU box), and the tuning code reads it to size persistent grids.

Reference: src/dew/nn/kernels/launches.py (launch / resource model), tables.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

SM_REGISTERS = 65536
SM_SHARED_BYTES = 233472          # 228 KB per SM, of which a CTA may use up to 227 KB
CTA_SHARED_MAX = 232448
SHARED_RESERVED_PER_CTA = 1024
SM_TMEM_COLUMNS = 512
SM_THREADS = 2048
SM_CTAS = 32
REGISTER_ALLOC_UNIT = 256         # registers are allocated per warp in units of 256


@dataclass(frozen=True)
class Launch:
    threads: int
    dynamic_smem: int = 0
    tmem_columns: int = 0


@dataclass(frozen=True)
class Occupancy:
    ctas_per_sm: int
    limiter: str
    by_registers: int
    by_shared: int
    by_tmem: int
    by_threads: int


def occupancy(registers: int, launch: Launch, static_smem: int = 0) -> Occupancy:
    warps = (launch.threads + 31) // 32
    regs_per_warp = (registers * 32 + REGISTER_ALLOC_UNIT - 1) // REGISTER_ALLOC_UNIT * REGISTER_ALLOC_UNIT
    by_regs = SM_REGISTERS // max(1, regs_per_warp * warps)
    smem = launch.dynamic_smem + static_smem + SHARED_RESERVED_PER_CTA
    by_smem = SM_SHARED_BYTES // smem if smem > 0 else SM_CTAS
    by_tmem = SM_TMEM_COLUMNS // launch.tmem_columns if launch.tmem_columns else SM_CTAS
    by_threads = SM_THREADS // max(1, launch.threads)
    limits = {"registers": by_regs, "shared memory": by_smem, "tensor memory": by_tmem, "threads": by_threads, "CTA slots": SM_CTAS}
    limiter = min(limits, key=limits.get)
    return Occupancy(max(0, limits[limiter]), limiter, by_regs, by_smem, by_tmem, by_threads)


# launch shapes of the tensor-core kernels (threads, dynamic shared memory, tensor-memory columns), as their launchers set them
LAUNCHES: Dict[str, Launch] = {
    "gemm_bf16_kernel": Launch(192, 4 * 49152 + 1280, 512),
    "gemm_pair_kernel": Launch(192, 6 * 32768 + 1280, 512),
    "gemm_mx_kernel": Launch(320, 5 * 40960 + 1280, 512),
    "flash_fwd_kernel": Launch(320, 229376 + 2560, 512),
    "flash_dq_kernel": Launch(320, 2 * 32768 + 5 * 2 * 16384 + 1280, 512),
    "flash_dkv_kernel": Launch(320, 232448 - 64, 512),
    "paged_decode_tma_kernel": Launch(128, 100 * 1024, 0),
}


def kernel_occupancy(name_part: str, resources: Optional[Dict[Tuple[str, str], Dict[str, int]]] = None) -> Dict[str, Occupancy]:
    """Occupancy of every compiled instantiation whose symbol contains ``name_part`` (needs the ptxas logs of a build)."""
    from . import build as B
    res = resources if resources is not None else B.kernel_resources()
    launch = next((l for k, l in LAUNCHES.items() if k in name_part or name_part in k), None)
    out = {}
    for (f, sym), r in res.items():
        if name_part in sym and launch is not None:
            out[sym] = occupancy(r["registers"], launch)
    return out
