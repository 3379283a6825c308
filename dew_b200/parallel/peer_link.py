"""A link of peer-visible buffers over one process group for the small, latency-bound exchanges of sequence / vocabulary /
feature parallelism: ``exchange`` (push to one rank, collect from another: halos, state hand-overs and their backward passes)
and ``all_reduce`` (short fp32 vectors, sum or max: row statistics).  Both are ONE kernel over NVLink peer memory whose
16-byte stores carry their own arrival tag (``csrc/kernels/peer_ll.cu``); on CPU ranks, one rank, or tensors that do not fit
the link the same operations run through ``torch.distributed``.

Messages of a directed pair of ranks are matched by count (the k-th ``exchange`` that sends from a to b meets the k-th that
receives on b from a), so calls need no global order; ``all_reduce`` is called by every rank of the group, in the same order.

Reference: the ``ppermute`` / ``psum`` / ``pmax`` of src/dew/nn/linear.py:696-781, src/dew/nn/local_attention.py:307,
src/dew/nn/kernels/recurrence_algebra.py:367-370, src/dew/objectives/lm/chunked.py:1143-1228, src/dew/nn/norms.py:429.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import library as L
from .symm import SymmetricBuffer

REGIONS = 2


class PeerLink:
    def __init__(self, group=None, max_bytes: int = 16 << 20, device=None, wait_limit_s: float = 60.0, max_reduce_floats: int = 1 << 18):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.max_bytes = (max_bytes + 15) // 16 * 16
        self.limit_ns = int(wait_limit_s * 1e9)
        self.fused = self.device.type == "cuda" and self.world > 1
        if self.fused:
            # [region][sender][2 * max_bytes] on every rank; acknowledgement words acks[reader] on every rank
            # the reductions have areas, tags and acknowledgement words of their own (words 8..15), after the exchange areas
            self.area = 2 * self.max_bytes
            self.reduce_area = (max_reduce_floats + 1) // 2 * 16
            self.reduce_base = REGIONS * self.world * self.area
            self.buf = SymmetricBuffer((self.reduce_base + REGIONS * self.world * self.reduce_area) // 4, torch.int32, self.device, group, zero=True)
            self.acks = SymmetricBuffer(64, torch.int32, self.device, group, zero=True)
            self.leave = torch.zeros(2, dtype=torch.int32, device=self.device)
            self.sent = [0] * self.world            # messages sent to each rank / received from each rank so far
            self.received = [0] * self.world
            self.reduce_tag = 0
            self.reduce_last = [0] * REGIONS

    def _global(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    # ------------------------------------------------------------------ point to point
    def exchange(self, x: Optional[torch.Tensor], to: Optional[int], frm: Optional[int], like: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Send ``x`` to rank ``to`` (None: nobody) and return what rank ``frm`` sent (None: nobody -> returns None).  ``like``
        gives the shape / dtype of what is received when nothing is sent.  Sender and receiver must pass equal byte counts."""
        ref = x if x is not None else like
        if to is not None and not 0 <= to < self.world:
            to = None
        if frm is not None and not 0 <= frm < self.world:
            frm = None
        out = torch.empty_like(ref, memory_format=torch.contiguous_format) if frm is not None else None
        if to is None and frm is None:
            return None
        nbytes = ref.numel() * ref.element_size()
        if self.fused and ref.is_cuda and nbytes % 16 == 0 and nbytes <= self.max_bytes:
            send_tag = recv_tag = need = 0
            if to is not None:
                self.sent[to] += 1
                send_tag = self.sent[to]
                need = max(0, send_tag - REGIONS)               # the message that last used this area must have been read
            if frm is not None:
                self.received[frm] += 1
                recv_tag = self.received[frm]
            xc = x.contiguous() if to is not None else None
            send_off = ((send_tag % REGIONS) * self.world + self.rank) * self.area
            recv_off = ((recv_tag % REGIONS) * self.world + (frm if frm is not None else 0)) * self.area
            L.check(L.load().dewb_peer_exchange(self.buf.ptr_array(), self.acks.ptr_array(), L.ptr(xc), L.ptr(out), ctypes.c_longlong(nbytes),
                                                ctypes.c_int(self.rank), ctypes.c_int(self.world), ctypes.c_int(-1 if to is None else to),
                                                ctypes.c_int(-1 if frm is None else frm), ctypes.c_uint(send_tag), ctypes.c_uint(recv_tag), ctypes.c_uint(need),
                                                ctypes.c_longlong(send_off), ctypes.c_longlong(recv_off), L.ptr(self.leave[:1]),
                                                ctypes.c_ulonglong(self.limit_ns), L.ptr(L.status(self.device)), L.stream_ptr()),
                    "peer_exchange")
            L.count_launches()
            return out
        ops_ = []
        if to is not None:
            ops_.append(dist.P2POp(dist.isend, x.contiguous(), self._global(to), self.group))
        if frm is not None:
            ops_.append(dist.P2POp(dist.irecv, out, self._global(frm), self.group))
        for w in dist.batch_isend_irecv(ops_):
            w.wait()
        return out

    # ------------------------------------------------------------------ short reductions
    def all_reduce(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """Sum or maximum over the ranks of a short fp32 tensor (a new tensor; the same on every rank)."""
        if self.world == 1:
            return x.clone()
        n = x.numel()
        if self.fused and x.is_cuda and x.dtype == torch.float32 and (n + 1) // 2 * 16 <= self.reduce_area:
            self.reduce_tag += 1
            region = self.reduce_tag % REGIONS
            need, self.reduce_last[region] = self.reduce_last[region], self.reduce_tag
            xc = x.contiguous()
            out = torch.empty_like(xc)
            L.check(L.load().dewb_allreduce_small(self.buf.ptr_array(), self.acks.ptr_array(8 * 4), L.ptr(xc), L.ptr(out), ctypes.c_longlong(n),
                                                  ctypes.c_int(self.rank), ctypes.c_int(self.world), ctypes.c_uint(self.reduce_tag), ctypes.c_uint(need),
                                                  ctypes.c_longlong(self.reduce_base + region * self.world * self.reduce_area),
                                                  ctypes.c_longlong(self.reduce_area), ctypes.c_int(0 if op == "sum" else 1), L.ptr(self.leave[1:]),
                                                  ctypes.c_ulonglong(self.limit_ns), L.ptr(L.status(self.device)), L.stream_ptr()),
                    "allreduce_small")
            L.count_launches()
            return out.view(x.shape)
        y = x.clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX, group=self.group)
        return y
