"""Symmetric (peer-mapped) device memory: a buffer allocated identically on every rank of a group whose per-rank
base addresses are known to all, so a kernel on one GPU can load from / store to any peer over NVLink.

The mapping itself (``cuMemCreate`` + fabric / fd handle exchange) is PyTorch's ``torch.distributed._symmetric_memory``;
everything that *uses* the peer pointers is this library's own kernels (``csrc/kernels/fsdp_comm.cu`` ...).
On one process, or on CPU ranks, a plain tensor stands in (world 1 has no peers).
"""
from __future__ import annotations

import os
from typing import List, Optional

# No rank of this library is ever bound to an NVLink multicast (NVLS) object: the kernels here use plain peer loads and
# stores, and a rank that exits while its memory is bound to a multicast object can raise NVLink faults on its peers'
# GPUs.  PyTorch reads this switch when it creates its first symmetric-memory block, i.e. after this import.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

import torch
import torch.distributed as dist


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, device, group: Optional[dist.ProcessGroup] = None,
                 zero: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and (group is not None or dist.get_world_size() > 1)) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.handle = None
        dev = torch.device(device)
        if self.world == 1 or dev.type != "cuda":
            self.tensor = torch.zeros(numel, dtype=dtype, device=dev) if zero else torch.empty(numel, dtype=dtype, device=dev)
            self.ptrs: List[int] = [self.tensor.data_ptr()]
            self.multicast_ptr = 0
        else:
            import torch.distributed._symmetric_memory as sm
            g = group if group is not None else dist.group.WORLD
            try:
                sm.enable_symm_mem_for_group(g.group_name)
            except Exception:
                pass
            self.tensor = sm.empty(numel, dtype=dtype, device=dev)
            self.handle = sm.rendezvous(self.tensor, g)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
            self.multicast_ptr = 0          # multicast mappings are switched off (see the top of this file)
            if zero:
                self.tensor.zero_()
            torch.cuda.synchronize(dev)
            dist.barrier(group=g)

    def ptr_array(self, offset_bytes: int = 0):
        """ctypes array of the W base addresses (+ offset), in rank order."""
        import ctypes
        return (ctypes.c_ulonglong * 8)(*([p + offset_bytes for p in self.ptrs] + [0] * (8 - len(self.ptrs))))

    def own_ptr_array(self, offset_bytes: int = 0):
        """ctypes array holding only this rank's base address (for kernels run with a world of one)."""
        import ctypes
        return (ctypes.c_ulonglong * 8)(*([self.tensor.data_ptr() + offset_bytes] + [0] * 7))

    def peer(self, rank: int, numel: Optional[int] = None, offset: int = 0) -> torch.Tensor:
        """A tensor view of ``rank``'s buffer (for host-side checks; kernels take ``ptr_array``)."""
        if self.handle is None:
            return self.tensor[offset: None if numel is None else offset + numel]
        n = self.tensor.numel() - offset if numel is None else numel
        return self.handle.get_buffer(rank, (n,), self.tensor.dtype, offset)
