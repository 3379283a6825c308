"""Page ledger for the paged KV cache: free list, reference counts and a chained-hash prefix cache.

A full page of prompt tokens is named by ``hash(previous page's name, its tokens)`` (the vLLM-style chain), so a new
request whose prompt starts with pages already in the pool re-uses them instead of recomputing; pages no request
references stay cached until the pool needs them back (least recently released first).
Parity: src/dew/inference/pages.py (chained-hash prefix cache + host tier), src/dew/inference/serving.py:415-590
(``PagedRows.seat``: page ledger, prefix reuse).
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


def chain_hash(previous: bytes, tokens: Sequence[int]) -> bytes:
    h = hashlib.sha256(previous)
    h.update(b",".join(str(int(t)).encode() for t in tokens))
    return h.digest()[:16]


class OutOfPages(RuntimeError):
    pass


@dataclass
class Seat:
    pages: List[int]            # the row's page table, in order
    reused_tokens: int          # prompt tokens already present in re-used pages (need no prefill)


class HostTier:
    """Evicted prefix pages kept in pinned host memory: when the device pool takes back a cached page, its keys and values (every
    layer's) are copied to a host slot under the page's chain hash; a later prompt with that prefix copies them back into a fresh
    device page instead of recomputing them.  Slots are recycled least recently used first.  The copies are issued on the
    current stream, so they are ordered against the kernels that wrote the page before and overwrite it after."""

    def __init__(self, store, slots: int):
        import torch
        self.store, self.slots = store, slots
        pin = store.device.type == "cuda"
        shape = (slots, store.layers, store.page_size, store.kv_heads, store.head_dim)
        self.k = torch.zeros(shape, dtype=store.k.dtype, pin_memory=pin)
        self.v = torch.zeros(shape, dtype=store.v.dtype, pin_memory=pin)
        quantized = store.k_scale is not None
        self.k_scale = torch.ones(shape[:-1], dtype=torch.float32, pin_memory=pin) if quantized else None
        self.v_scale = torch.ones(shape[:-1], dtype=torch.float32, pin_memory=pin) if quantized else None
        self.slot_of: "OrderedDict[bytes, int]" = OrderedDict()           # oldest first
        self.free: List[int] = list(range(slots - 1, -1, -1))
        self.spilled = self.fetched = 0

    def has(self, name: bytes) -> bool:
        return name in self.slot_of

    def spill(self, page: int, name: bytes) -> None:
        if self.slots <= 0:
            return
        if name in self.slot_of:
            self.slot_of.move_to_end(name)
            return
        slot = self.free.pop() if self.free else self.slot_of.popitem(last=False)[1]
        st = self.store
        self.k[slot].copy_(st.k[:, page], non_blocking=True)
        self.v[slot].copy_(st.v[:, page], non_blocking=True)
        if self.k_scale is not None:
            self.k_scale[slot].copy_(st.k_scale[:, page], non_blocking=True)
            self.v_scale[slot].copy_(st.v_scale[:, page], non_blocking=True)
        self.slot_of[name] = slot
        self.spilled += 1

    def fetch(self, name: bytes, page: int) -> bool:
        slot = self.slot_of.get(name)
        if slot is None:
            return False
        self.slot_of.move_to_end(name)
        st = self.store
        st.k[:, page].copy_(self.k[slot], non_blocking=True)
        st.v[:, page].copy_(self.v[slot], non_blocking=True)
        if self.k_scale is not None:
            st.k_scale[:, page].copy_(self.k_scale[slot], non_blocking=True)
            st.v_scale[:, page].copy_(self.v_scale[slot], non_blocking=True)
        self.fetched += 1
        return True


class PageLedger:
    def __init__(self, pages: int, page_size: int, prefix_cache: bool = True, host: Optional[HostTier] = None):
        self.pages, self.page_size, self.prefix_cache = pages, page_size, prefix_cache
        self.host = host
        self.host_hits = 0
        self.free: List[int] = list(range(pages - 1, -1, -1))
        self.refs: Dict[int, int] = {}
        self.name_of: Dict[int, bytes] = {}                 # page -> chain hash (only full prompt pages)
        self.page_of: Dict[bytes, int] = {}
        self.idle: "OrderedDict[int, None]" = OrderedDict()  # cached pages with no references, oldest first
        self.hits = 0
        self.lookups = 0

    def available(self) -> int:
        return len(self.free) + len(self.idle)

    def _take(self) -> int:
        if self.free:
            return self.free.pop()
        if self.idle:
            page, _ = self.idle.popitem(last=False)          # evict the least recently released cached page
            name = self.name_of.pop(page, None)
            if name is not None:
                self.page_of.pop(name, None)
                if self.host is not None:
                    self.host.spill(page, name)              # its contents move to the host tier before the page is reused
            return page
        raise OutOfPages("the KV page pool is exhausted")

    def seat(self, prompt: Sequence[int], total_tokens: int) -> Seat:
        """Pages for a row that will hold ``total_tokens`` (prompt + generation budget), re-using cached prefix pages."""
        need = (total_tokens + self.page_size - 1) // self.page_size
        pages: List[int] = []
        reused = 0
        prev = b""
        full_prompt_pages = len(prompt) // self.page_size
        if self.prefix_cache:
            for i in range(full_prompt_pages):
                # never re-use the page holding the prompt's last token: its logits must be computed
                if (i + 1) * self.page_size >= len(prompt):
                    break
                name = chain_hash(prev, prompt[i * self.page_size:(i + 1) * self.page_size])
                self.lookups += 1
                page = self.page_of.get(name)
                if page is None:
                    if self.host is None or not self.host.has(name) or self.available() == 0:
                        break
                    page = self._take()                      # bring the page back from the host tier under its old name
                    self.host.fetch(name, page)
                    self.page_of[name], self.name_of[page] = page, name
                    self.host_hits += 1
                self.hits += 1
                self.idle.pop(page, None)
                self.refs[page] = self.refs.get(page, 0) + 1
                pages.append(page)
                reused += self.page_size
                prev = name
        if need - len(pages) > self.available():
            for p in pages:
                self._release_one(p)
            raise OutOfPages(f"need {need - len(pages)} pages, {self.available()} available")
        while len(pages) < need:
            p = self._take()
            self.refs[p] = 1
            pages.append(p)
        return Seat(pages, reused)

    def publish(self, prompt: Sequence[int], pages: Sequence[int]) -> None:
        """After a prompt's prefill: name its full pages so later requests can re-use them."""
        if not self.prefix_cache:
            return
        prev = b""
        for i in range(len(prompt) // self.page_size):
            name = chain_hash(prev, prompt[i * self.page_size:(i + 1) * self.page_size])
            page = pages[i]
            if name not in self.page_of and page not in self.name_of:
                self.page_of[name] = page
                self.name_of[page] = name
            prev = name

    def _release_one(self, page: int) -> None:
        n = self.refs.get(page, 0) - 1
        if n > 0:
            self.refs[page] = n
            return
        self.refs.pop(page, None)
        if page in self.name_of:
            self.idle[page] = None           # keep its contents cached
        else:
            self.free.append(page)

    def release(self, pages: Sequence[int]) -> None:
        for p in pages:
            self._release_one(p)
