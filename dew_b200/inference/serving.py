"""Continuous-batching server: slots, admission with chunked prefill, paged KV cache with prefix re-use, tickets that
stream tokens and record time-to-first-token, and a decode loop whose host read is one step behind the device.

Parity: src/dew/inference/serving.py (``Server.from_task`` :889-1010, ``submit`` :1075, ``step`` :1262-1324, ``run``
:1465, ``_admit`` :1572, ``_settle`` :1676, ``Ticket`` :204-240), serving_kernel.py (mixed prefill + decode step).
Every process of a tensor-parallel group runs the same schedule on the same requests (it is deterministic), so no
cross-rank agreement is needed inside a step; the model's collectives synchronise the devices.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence

import torch

from ..nn.kv_cache import KVCache, KVStore
from ..sampling.text import Sampling, transform_logits
from ..utils import keys as K
from .pages import HostTier, OutOfPages, PageLedger


@dataclass
class Ticket:
    """A submitted request: tokens arrive as they are settled; ``first_token_time`` is TTFT in seconds."""
    prompt: List[int]
    max_new_tokens: int
    key: int = 0
    sampling: Optional[Sampling] = None
    on_token: Optional[Callable[[int], None]] = None
    tokens: List[int] = field(default_factory=list)
    submitted: float = 0.0
    first_token_time: Optional[float] = None
    finished_time: Optional[float] = None
    done: bool = False
    terminated: bool = False
    error: Optional[BaseException] = None

    def result(self) -> List[int]:
        if self.error is not None:
            raise self.error
        return self.tokens


@dataclass
class _Row:
    ticket: Ticket
    pages: List[int]
    prefilled: int = 0          # prompt tokens already in the cache
    generated: int = 0
    pending_first: bool = False


class Server:
    def __init__(self, model, variables=None, *, slots: int, capacity: int, kv_cache: Optional[KVCache] = None,
                 chunk: Optional[int] = None, prefix_cache: bool = True, decode_steps: int = 1, sampling: Optional[Sampling] = None,
                 tokenizer=None, prefill_budget: Optional[int] = None, cuda_graph: bool = False, clock: Callable[[], float] = time.perf_counter,
                 host_pages: int = 0):
        self.model, self.variables, self.tokenizer = model, variables, tokenizer
        self.slots, self.capacity = slots, capacity
        limit = getattr(getattr(model, "config", None), "max_seq_len", None)
        if limit is not None and capacity > limit:
            raise ValueError(f"row capacity {capacity} exceeds the model's max_seq_len {limit} (its rotary tables end there)")
        spec = kv_cache if isinstance(kv_cache, KVCache) else KVCache(page_size=kv_cache if isinstance(kv_cache, int) else 16)
        if spec.page_size is None:
            spec = KVCache(spec.quantized, capacity, spec.pages, spec.groups, spec.offloaded)
        pages_per_row = (capacity + spec.page_size - 1) // spec.page_size
        pool = spec.pages or slots * pages_per_row
        self.spec = KVCache(spec.quantized, spec.page_size, pool, spec.groups, spec.offloaded)
        cfg = model.config
        p = next(model.parameters())
        hd = cfg.head_dim or cfg.emb_features // cfg.num_heads
        kvh = getattr(model, "local_kv_heads", None) or (cfg.num_kv_heads or cfg.num_heads)
        self.store = KVStore(self.spec, cfg.num_layers, slots, capacity, kvh, hd, p.dtype, p.device)
        self.host_tier = HostTier(self.store, host_pages) if host_pages > 0 and prefix_cache else None
        self.ledger = PageLedger(pool, self.spec.page_size, prefix_cache, self.host_tier)
        self.chunk = chunk or 512
        self.prefill_budget = prefill_budget or 8 * self.chunk     # prompt tokens admitted per step (keeps decode latency bounded)
        self.decode_steps = decode_steps
        self.sampling = sampling or Sampling(temperature=0.0)
        self.rows: List[Optional[_Row]] = [None] * slots
        self.queue: Deque[Ticket] = deque()
        self.device = p.device
        self.clock = clock
        self.last_tokens = torch.zeros(slots, dtype=torch.long, device=self.device)      # device-resident draws
        self._pending: Optional[tuple] = None                                            # (tokens on host (async), rows snapshot, event)
        self.cuda_graph = cuda_graph and self.device.type == "cuda"
        self._graph = None
        self.steps = 0
        self.wait_s = 0.0
        self.decoded_tokens = 0
        if variables is None:
            self._call = lambda t, **kw: model(t, **kw)
        else:
            from ..utils.trees import variables_for_call
            named = variables_for_call(model, variables)
            self._call = lambda t, **kw: torch.func.functional_call(model, named, (t,), kw)

    # ------------------------------------------------------------------ construction / API
    @classmethod
    def from_task(cls, task, *, slots: int, capacity: int, admission=None, kv_cache=None, chunk=None, prefix_cache=None,
                  host_pages: int = 0, decode_steps: int = 1, cuda_graph: bool = False) -> "Server":
        return cls(task.model, task.variables, slots=slots, capacity=capacity, kv_cache=kv_cache if kv_cache is not None else task.kv_cache,
                   chunk=chunk, prefix_cache=True if prefix_cache is None else bool(prefix_cache), decode_steps=decode_steps, host_pages=host_pages,
                   sampling=task.sampling, tokenizer=task.tokenizer, cuda_graph=cuda_graph)

    def submit(self, prompt, max_new_tokens: int, key: int = 0, sampling: Optional[Sampling] = None, on_token=None) -> Ticket:
        if isinstance(prompt, str):
            prompt = self.tokenizer.encode(prompt)
        prompt = [int(t) for t in prompt]
        if len(prompt) + max_new_tokens > self.capacity:
            raise ValueError(f"prompt of {len(prompt)} tokens + {max_new_tokens} new exceeds the row capacity {self.capacity}")
        t = Ticket(prompt, max_new_tokens, key, sampling, on_token, submitted=self.clock())
        self.queue.append(t)
        return t

    @property
    def occupancy(self) -> int:
        return sum(r is not None for r in self.rows)

    @property
    def queued(self) -> int:
        return len(self.queue)

    @property
    def busy(self) -> bool:
        return self.occupancy > 0 or bool(self.queue) or self._pending is not None

    def fail(self, exc: BaseException) -> None:
        for r in self.rows:
            if r is not None:
                r.ticket.error, r.ticket.done = exc, True
        for t in self.queue:
            t.error, t.done = exc, True
        self.queue.clear()
        self.rows = [None] * self.slots

    def reload(self, variables) -> None:
        self.variables = variables
        from ..utils.trees import variables_for_call
        named = variables_for_call(self.model, variables)
        self._call = lambda t, **kw: torch.func.functional_call(self.model, named, (t,), kw)
        self._graph = None

    def __call__(self, prompts: Sequence[Any], max_new_tokens: int = 32) -> List[List[int]]:
        tickets = [self.submit(p, max_new_tokens) for p in prompts]
        self.run()
        return [t.result() for t in tickets]

    def run(self, max_steps: Optional[int] = None) -> None:
        n = 0
        while self.busy and (max_steps is None or n < max_steps):
            self.step()
            n += 1

    # ------------------------------------------------------------------ one step
    def step(self) -> None:
        self._seat()
        self._prefill()
        launched = self._decode()
        self._settle(keep_latest=launched)
        self.steps += 1

    def _seat(self) -> None:
        if not self.queue:
            return
        for slot in range(self.slots):
            if self.rows[slot] is not None or not self.queue:
                continue
            t = self.queue[0]
            try:
                seat = self.ledger.seat(t.prompt, len(t.prompt) + t.max_new_tokens)
            except OutOfPages:
                break
            self.queue.popleft()
            table = self.store.page_table[slot]
            table[: len(seat.pages)] = torch.tensor(seat.pages, dtype=torch.int32, device=self.device)
            self.rows[slot] = _Row(t, seat.pages, prefilled=seat.reused_tokens)

    def _prefill(self) -> None:
        """Chunked prefill: every row still reading its prompt advances by up to ``chunk`` tokens; rows are batched and
        padded to the longest chunk of the step."""
        waiting = [(s, r) for s, r in enumerate(self.rows) if r is not None and r.prefilled < len(r.ticket.prompt)]
        if not waiting:
            return
        todo, budget = [], self.prefill_budget
        for s, r in sorted(waiting, key=lambda sr: sr[1].ticket.submitted):
            take = min(self.chunk, len(r.ticket.prompt) - r.prefilled)
            if todo and take > budget:
                break
            todo.append((s, r))
            budget -= take
        # rows that share a start offset of 0 can use the fast path; others attend to their cached prefix
        groups: Dict[int, list] = {}
        for s, r in todo:
            groups.setdefault(r.prefilled, []).append((s, r))
        for start, members in groups.items():
            width = min(self.chunk, max(len(r.ticket.prompt) - start for _, r in members))
            if self.device.type == "cuda" and width > 1:
                # a multiple of 128 keeps the chunk on the flash kernels and the set of shapes small; the pad positions are -1
                # (not written to the cache, never attended to by the real positions before them)
                width = (width + 127) // 128 * 128
            # the batch is assembled on the host and crosses to the device once
            ids_h = torch.zeros(len(members), width, dtype=torch.long)
            pos_h = torch.full((len(members), width), -1, dtype=torch.long)
            last = []
            longest = 0
            for i, (s, r) in enumerate(members):
                piece = r.ticket.prompt[start:start + width]
                ids_h[i, :len(piece)] = torch.tensor(piece, dtype=torch.long)
                pos_h[i, :len(piece)] = torch.arange(start, start + len(piece))
                last.append(len(piece) - 1)
                longest = max(longest, len(piece))
            ids, pos = ids_h.to(self.device, non_blocking=True), pos_h.to(self.device, non_blocking=True)
            slots = torch.tensor([s for s, _ in members], device=self.device)
            self.store.chunk_span = (start, start + longest)
            with torch.no_grad():
                # the head runs only on each row's last position (the only logits a prefill chunk can need)
                if hasattr(self.model, "logits"):
                    hidden = self._call(ids, positions=pos, cache=self.store.select(slots), return_hidden=True)
                    picked = hidden[torch.arange(len(members), device=self.device), torch.tensor(last, device=self.device)]
                    last_logits = self.model.logits(picked)
                else:
                    full = self._call(ids, positions=pos, cache=self.store.select(slots))
                    last_logits = full[torch.arange(len(members), device=self.device), torch.tensor(last, device=self.device)]
            self.store.select(None)
            self.store.chunk_span = None
            for i, (s, r) in enumerate(members):
                r.prefilled += last[i] + 1
                if r.prefilled >= len(r.ticket.prompt):
                    self.ledger.publish(r.ticket.prompt, r.pages)
                    tok = self._draw(last_logits[i][None], r, 0)
                    self.last_tokens[s] = tok
                    r.pending_first = True

    def _draw(self, logits: torch.Tensor, row: _Row, step: int) -> torch.Tensor:
        s = row.ticket.sampling or self.sampling
        if s.greedy:
            return logits[0].argmax(-1)
        if logits.is_cuda:
            from ..ops import sample as S
            from ..sampling.text import plain_filters
            if plain_filters(s) and S.kernel_ok(logits):
                # temperature and the top-k / min-p / top-p thresholds inside the sampling kernel; the uniform comes from the row's key
                g = K.generator(K.fold_in(K.fold_in(K.key(row.ticket.key), "draw"), step), "cpu")
                return S.sample_rows(logits, torch.rand(1, generator=g), max(s.temperature, 1e-6), s.top_k, s.top_p, s.min_p)[0]
        hist = torch.tensor([row.ticket.prompt + row.ticket.tokens], device=logits.device)
        x = transform_logits(logits, hist, torch.tensor([hist.shape[1]], device=logits.device), s, step)
        p = torch.softmax(x, -1)[0]
        g = K.generator(K.fold_in(K.fold_in(K.key(row.ticket.key), "draw"), step), "cpu")
        return torch.multinomial(p.cpu(), 1, generator=g)[0].to(logits.device)

    def _decode_program(self, greedy: bool) -> None:
        """Device work of one decode step, on static buffers (``last_tokens``, ``_in_pos``, ``_prev``) so that it can be
        captured once into a CUDA graph and replayed."""
        self._prev.copy_(self.last_tokens)
        with torch.no_grad():
            hidden = self._call(self.last_tokens[:, None], positions=self._in_pos[:, None], cache=self.store.select(None),
                                return_hidden=True)[:, 0]
            if greedy:
                nxt = self.model.next_tokens_greedy(hidden)
            else:
                self._logits = self.model.logits(hidden)
                nxt = self._logits.argmax(-1)
        self.last_tokens.copy_(torch.where(self._in_pos >= 0, nxt, self.last_tokens))

    def _decode(self) -> bool:
        """One decode step for every row that has its prompt in the cache. Input tokens are the device-resident draws
        of the previous step; the host has not read them yet."""
        active = [(s, r) for s, r in enumerate(self.rows) if r is not None and r.prefilled >= len(r.ticket.prompt)]
        if not active:
            return False
        if not hasattr(self, "_in_pos"):
            self._in_pos = torch.full((self.slots,), -1, dtype=torch.long, device=self.device)
            self._prev = torch.zeros(self.slots, dtype=torch.long, device=self.device)
            # The device runs behind the host, so a pinned staging buffer may still be waiting to be copied when the
            # next step is prepared: rotate over more buffers than steps can be in flight.
            self._host_ring = [torch.full((self.slots,), -1, dtype=torch.long, pin_memory=self.device.type == "cuda") for _ in range(8)]
            self._ring_events = [None] * 8
            self._ring_at = 0
        self._ring_at = (self._ring_at + 1) % len(self._host_ring)
        if self._ring_events[self._ring_at] is not None:
            self._ring_events[self._ring_at].synchronize()
        self._host_pos = self._host_ring[self._ring_at]
        # one list, written into the pinned buffer in one assignment (per-element tensor writes cost microseconds each)
        vals = [-1] * self.slots
        greedy = True
        default_greedy = self.sampling.greedy
        for s, r in active:
            t = r.ticket
            if r.generated + 1 < t.max_new_tokens:
                vals[s] = len(t.prompt) + r.generated
            greedy = greedy and (default_greedy if t.sampling is None else t.sampling.greedy)
        self._host_pos.numpy()[:] = vals
        any_live = max(vals) >= 0
        self._in_pos.copy_(self._host_pos, non_blocking=True)
        if self.device.type == "cuda":
            e = torch.cuda.Event()
            e.record()
            self._ring_events[self._ring_at] = e
        if any_live:
            if self.cuda_graph and greedy:
                if self._graph is None:
                    self._decode_program(True)                      # warm-up (allocations, lazy initialisation)
                    torch.cuda.synchronize()
                    # the warm-up advanced the cache by one token for every row; replaying the same positions
                    # rewrites the same slots with the same values, so the cache stays consistent
                    self.last_tokens.copy_(self._prev)
                    self._graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(self._graph):
                        self._decode_program(True)
                    self.last_tokens.copy_(self._prev)
                self._graph.replay()
            else:
                self._decode_program(greedy)
                if not greedy:
                    for s, r in active:
                        if self._host_pos[s] >= 0 and not (r.ticket.sampling or self.sampling).greedy:
                            self.last_tokens[s] = self._draw(self._logits[s][None], r, r.generated + 1)
        else:
            self._prev.copy_(self.last_tokens)
        snapshot = active
        # hand the tokens that were the *input* of this step to the host, asynchronously
        host = torch.empty(self.slots, dtype=torch.long, pin_memory=self.device.type == "cuda")
        host.copy_(self._prev, non_blocking=True)
        ev = torch.cuda.Event() if self.device.type == "cuda" else None
        if ev is not None:
            ev.record()
        self._queue_settle(host, snapshot, ev)
        for s, r in active:
            r.generated += 1
        return True

    def _queue_settle(self, host, snapshot, ev) -> None:
        self._later = getattr(self, "_later", deque())
        self._later.append((host, snapshot, ev))

    def _settle(self, keep_latest: bool) -> None:
        """Read draws whose copy has landed: all but the newest while the device is still busy with it."""
        later = getattr(self, "_later", deque())
        keep = 1 if (keep_latest and self.device.type == "cuda") else 0
        while len(later) > keep:
            host, snapshot, ev = later.popleft()
            if ev is not None:
                t_wait = time.perf_counter()
                ev.synchronize()
                self.wait_s += time.perf_counter() - t_wait       # time the host stood waiting for the device
            now = self.clock()
            toks = host.tolist()
            for s, r in snapshot:
                t = r.ticket
                if t.done:
                    continue
                tok = toks[s]
                t.tokens.append(tok)
                self.decoded_tokens += 1
                if t.first_token_time is None:
                    t.first_token_time = now - t.submitted
                if t.on_token is not None:
                    t.on_token(tok)
                samp = t.sampling or self.sampling
                if (samp.eos_token_ids and tok in samp.eos_token_ids) or len(t.tokens) >= t.max_new_tokens:
                    t.terminated = bool(samp.eos_token_ids and tok in samp.eos_token_ids)
                    t.done, t.finished_time = True, now
                    if self.rows[s] is r:
                        self.ledger.release(r.pages)
                        self.rows[s] = None
        self._pending = None if not later else later[-1]
