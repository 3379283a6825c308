"""KV cache: dense or paged pools, optional int8 / fp8-e4m3 storage, decode attention over the pages.

Parity: src/dew/nn/kv_cache.py (``KVCache`` spec :362-408 - ``quantized``, ``page_size``, ``pages``, ``groups``,
``offloaded``; ``quantize`` / ``dequantize`` :411-446 per-token-per-head absmax scales; ``hadamard`` :465-479;
``KVStore.write / attend / decode`` :787-1180; pool layout :1297-1320; ``gather_cache_rows`` :1686).
Pool layout here: ``[layers, pages, page_size, kv_heads, head_dim]`` for keys and for values, a page table
``[rows, max_pages]`` and ``lengths [rows]``; a dense cache is the special case of one page per row.
"""
from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import ops
from ..ops import library as L

LIMITS = {"int8": 127.0, "float8_e4m3fn": 448.0}
KINDS = {None: 0, "int8": 1, "float8_e4m3fn": 2}


@dataclass(frozen=True)
class KVCache:
    quantized: Optional[str] = None           # None | "int8" | "float8_e4m3fn"
    page_size: Optional[int] = None           # None: dense ("whole") rows
    pages: Optional[int] = None               # pool size; default rows * pages_per_row
    groups: int = 1
    offloaded: bool = False

    def __post_init__(self):
        if self.quantized not in KINDS:
            raise ValueError(f"quantized must be one of {list(KINDS)}, got {self.quantized!r}")


def hadamard(x: torch.Tensor) -> torch.Tensor:
    """Fast Walsh-Hadamard transform over the last axis (a power of two), orthonormal; spreads outliers before int8."""
    n = x.shape[-1]
    assert n & (n - 1) == 0
    y = x.float().reshape(-1, n)
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        y = torch.stack([y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]], 2).reshape(-1, n)
        h *= 2
    return (y / math.sqrt(n)).reshape(x.shape)


def quantize(x: torch.Tensor, kind: str) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token-per-head: ``scale = absmax / limit``; returns (stored values, fp32 scales ``[..., heads]``)."""
    limit = LIMITS[kind]
    amax = x.float().abs().amax(-1)
    scale = torch.where(amax > 0, amax / limit, torch.ones_like(amax))
    y = x.float() / scale[..., None]
    if kind == "int8":
        return y.round().clamp(-127, 127).to(torch.int8), scale
    return y.to(torch.float8_e4m3fn), scale


def dequantize(q: torch.Tensor, scale: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    return (q.float() * scale[..., None]).to(dtype)


def default_page_table(rows: int, pages_per_row: int, device=None) -> torch.Tensor:
    return torch.arange(rows * pages_per_row, dtype=torch.int32, device=device).reshape(rows, pages_per_row)


class KVStore:
    def __init__(self, spec: KVCache, layers: int, rows: int, max_len: int, kv_heads: int, head_dim: int,
                 dtype=torch.bfloat16, device="cpu"):
        self.spec = spec
        self.layers, self.rows, self.max_len, self.kv_heads, self.head_dim = layers, rows, max_len, kv_heads, head_dim
        self.page_size = spec.page_size or max_len
        self.max_pages = (max_len + self.page_size - 1) // self.page_size
        self.pages = spec.pages or rows * self.max_pages
        self.kind = KINDS[spec.quantized]
        store = {0: dtype, 1: torch.int8, 2: torch.float8_e4m3fn}[self.kind]
        # one page beyond the addressable pool: writes of padding positions land there, so that a write needs no data-dependent
        # shapes (and therefore no host synchronisation); no page table entry ever names it
        shape = (layers, self.pages + 1, self.page_size, kv_heads, head_dim)
        self.k = torch.zeros(shape, dtype=store, device=device)
        self.v = torch.zeros(shape, dtype=store, device=device)
        self.k_scale = torch.ones(shape[:-1], dtype=torch.float32, device=device) if self.kind else None
        self.v_scale = torch.ones(shape[:-1], dtype=torch.float32, device=device) if self.kind else None
        self.page_table = default_page_table(rows, self.max_pages, device) if spec.pages is None else \
            torch.zeros(rows, self.max_pages, dtype=torch.int32, device=device)
        self.lengths = torch.zeros(rows, dtype=torch.int32, device=device)
        self.dtype, self.device = dtype, torch.device(device)
        self.row_ids: Optional[torch.Tensor] = None      # rows of the store addressed by the batch rows of a call
        self._scratch = None
        self.chunk_span: Optional[Tuple[int, int]] = None      # (first position, one past the last) of the prefill chunk in flight, when the caller knows

    # ------------------------------------------------------------------ latent rows (multi-head latent attention)
    def latent(self, layer: int, width: int) -> torch.Tensor:
        """``[rows, max_len, width]`` per layer: what multi-head latent attention caches per token (its normalised KV latent
        and the shared rotary key) instead of per-head keys and values.  Allocated on first use."""
        bank = self.__dict__.setdefault("_latent", {})
        if layer not in bank:
            bank[layer] = torch.zeros(self.rows, self.max_len, width, dtype=self.dtype, device=self.device)
        return bank[layer]

    def write_latent(self, layer: int, values: torch.Tensor, positions: torch.Tensor) -> None:
        """``values [R, S, width]`` at ``positions [R, S]`` of the selected rows (negative positions are skipped)."""
        R, S = positions.shape
        buf = self.latent(layer, values.shape[-1])
        rows = self._rows(R)[:, None].expand(R, S)
        live = positions >= 0
        buf[rows[live], positions[live].long()] = values[live].to(buf.dtype)

    def read_latent(self, layer: int, width: int, length: int) -> torch.Tensor:
        """The selected rows' first ``length`` cached latents ``[R, length, width]``."""
        buf = self.latent(layer, width)
        rows = self._rows(self.rows if self.row_ids is None else self.row_ids.numel())
        return buf[rows, :length]

    # ------------------------------------------------------------------ addressing
    def select(self, row_ids: Optional[torch.Tensor]) -> "KVStore":
        """Batch row ``i`` of the next calls addresses store row ``row_ids[i]`` (None: identity)."""
        self.row_ids = None if row_ids is None else row_ids.to(self.device, torch.int64)
        return self

    def _rows(self, n: int) -> torch.Tensor:
        return torch.arange(n, device=self.device) if self.row_ids is None else self.row_ids

    def _slots(self, rows: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Flat pool token index (page * page_size + offset) for (row, position) pairs."""
        page = self.page_table[rows, (positions // self.page_size).long()].long()
        return page * self.page_size + (positions % self.page_size).long()

    # ------------------------------------------------------------------ writes
    def write(self, layer: int, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor) -> None:
        """Store ``k, v [R, S, Hkv, D]`` at ``positions [R, S]`` (negative positions are skipped)."""
        R, S = positions.shape
        rows = self._rows(R)[:, None].expand(R, S).reshape(-1)
        flat = positions.reshape(-1)
        live = flat >= 0
        slots = torch.where(live, self._slots(rows, flat.clamp_min(0)), self.pages * self.page_size)      # padding -> the spare page
        kk, vv = k.reshape(R * S, self.kv_heads, self.head_dim), v.reshape(R * S, self.kv_heads, self.head_dim)
        kp, vp = self.k[layer].reshape(-1, self.kv_heads, self.head_dim), self.v[layer].reshape(-1, self.kv_heads, self.head_dim)
        if self.kind:
            kq, ks = quantize(kk, self.spec.quantized)
            vq, vs = quantize(vv, self.spec.quantized)
            kp[slots], vp[slots] = kq, vq
            self.k_scale[layer].reshape(-1, self.kv_heads)[slots] = ks
            self.v_scale[layer].reshape(-1, self.kv_heads)[slots] = vs
        else:
            kp[slots], vp[slots] = kk.to(kp.dtype), vv.to(vp.dtype)

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor) -> None:
        """One token per row: ``k, v [R, Hkv, D]`` written at ``positions [R]``."""
        if L.use_cuda(k) and k.dtype == torch.bfloat16 and self.row_ids is None and k.shape[0] == self.rows:
            lib = L.load()
            # every temporary stays referenced until the launch is enqueued: a temporary released between two `L.ptr` calls hands
            # its block back to the allocator, and the next temporary of the same size would take (and overwrite) it
            kc, vc, pos32 = k.contiguous(), v.contiguous(), positions.to(torch.int32).contiguous()
            L.check(lib.dewb_kv_append(L.ptr(kc), L.ptr(vc), L.ptr(self.k[layer]), L.ptr(self.v[layer]),
                                       L.ptr(self.k_scale[layer] if self.kind else None),
                                       L.ptr(self.v_scale[layer] if self.kind else None), L.ptr(self.page_table),
                                       L.ptr(pos32), ctypes.c_int(k.shape[0]),
                                       ctypes.c_int(self.kv_heads), ctypes.c_int(self.head_dim), ctypes.c_int(self.page_size),
                                       ctypes.c_int(self.max_pages), ctypes.c_int(self.kind), L.stream_ptr()), "kv_append")
            L.count_launches()
            return
        self.write(layer, k[:, None], v[:, None], positions[:, None])

    # ------------------------------------------------------------------ the fused decode step
    def _step_ints(self, positions: torch.Tensor):
        """(positions, lengths) of a decode step as int32, computed once per step: every layer of a forward passes the same
        positions tensor, so the conversions and the ``where`` run for the first layer only."""
        key = (positions.data_ptr(), positions._version, tuple(positions.shape), torch.cuda.is_current_stream_capturing() if positions.is_cuda else False)
        cached = getattr(self, "_ints", None)
        if cached is not None and cached[0] == key:
            return cached[1], cached[2]
        pos32 = positions.to(torch.int32).contiguous()
        lens32 = torch.where(pos32 >= 0, pos32 + 1, torch.zeros_like(pos32))
        self._ints = (key, pos32, lens32)
        return pos32, lens32

    def can_decode_packed(self, qkv: torch.Tensor, Hq: int, softcap: float = 0.0) -> bool:
        return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and self.kind == 0 and self.row_ids is None
                and qkv.shape[0] == self.rows and self.head_dim == 128 and self.page_size % 64 == 0 and not softcap
                and Hq // self.kv_heads <= 8 and os.environ.get("DEWB_DECODE", "stream") == "stream"
                and hasattr(L.load(), "dewb_rope_append"))

    MIN_TILES = 4            # fewest 64-key tiles one CTA of the balanced decode kernel takes (bounds the parts a row is cut into)

    def _fused_decode(self, lib, layer: int, q, q_row_stride: int, lens32, R: int, Hq: int, D: int, window, sinks32, out) -> None:
        """The streamed paged-attention kernel finishing its rows itself.  Up to 1024 rows take the balanced persistent form
        (every CTA moves the same number of tiles, whatever the rows' lengths); more rows take one CTA per (row, head, chunk)."""
        longest = min(self.max_len, window) if window else self.max_len
        max_tiles = -(-longest // 64) + 1                                 # (+ 1: a window that straddles a tile boundary)
        persist = R <= 1024 and os.environ.get("DEWB_DECODE_PERSIST", "1") == "1"
        if persist:
            min_tiles = int(os.environ.get("DEWB_DECODE_MIN_TILES", self.MIN_TILES))
            splits = (max_tiles - 1) // min_tiles + 2
        else:
            chunk = 8
            splits = max(1, -(-max_tiles // chunk))
        n = R * Hq * splits
        if self._scratch is None or self._scratch[0].numel() < n:
            self._scratch = (torch.empty(n, dtype=torch.float32, device=q.device), torch.empty(n, dtype=torch.float32, device=q.device),
                             torch.empty(n * D, dtype=torch.float32, device=q.device))
        if getattr(self, "_arrivals", None) is None or self._arrivals.numel() < R * self.kv_heads:
            self._arrivals = torch.zeros(R * self.kv_heads, dtype=torch.int32, device=q.device)
        pm, pl, pa = self._scratch
        common = (L.ptr(q), L.ptr(self.k[layer]), L.ptr(self.v[layer]), ctypes.c_longlong(self.pages * self.page_size),
                  L.ptr(self.page_table), L.ptr(lens32), L.ptr(pm), L.ptr(pl), L.ptr(pa), L.ptr(self._arrivals), L.ptr(sinks32),
                  L.ptr(out), ctypes.c_int(R), ctypes.c_int(Hq), ctypes.c_int(self.kv_heads), ctypes.c_int(self.page_size),
                  ctypes.c_int(self.max_pages), ctypes.c_int(splits))
        if persist:
            if getattr(self, "_ctas", None) is None:
                self._ctas = 2 * torch.cuda.get_device_properties(q.device).multi_processor_count
            L.check(lib.dewb_paged_decode_persist(*common, ctypes.c_int(min_tiles), ctypes.c_float(1.0 / math.sqrt(D)),
                                                  ctypes.c_int(window or 0), ctypes.c_longlong(q_row_stride), ctypes.c_int(self._ctas),
                                                  L.ptr(L.status(q.device)), L.stream_ptr()), "paged_decode_persist")
        else:
            L.check(lib.dewb_paged_decode_fused(*common, ctypes.c_int(chunk), ctypes.c_float(1.0 / math.sqrt(D)),
                                                ctypes.c_int(window or 0), ctypes.c_longlong(q_row_stride),
                                                L.ptr(L.status(q.device)), L.stream_ptr()), "paged_decode_fused")
        L.count_launches()

    def decode_packed(self, layer: int, qkv: torch.Tensor, cos, sin, positions: torch.Tensor, Hq: int, window=None, sinks=None):
        """One decode step of a layer straight from the packed projection output ``qkv [R, Hq + 2 Hkv, D]``: one kernel rotates
        the query / key heads in place and appends the keys and values to the paged cache, then the streamed paged-attention
        kernel reads the queries where they are (row stride of the packed tensor).  Returns ``[R, Hq, D]``."""
        lib = L.load()
        R, H, D = qkv.shape
        pos32, lens32 = self._step_ints(positions)
        L.check(lib.dewb_rope_append(L.ptr(qkv), L.ptr(cos), L.ptr(sin), L.ptr(pos32), ctypes.c_int(R), ctypes.c_int(Hq),
                                     ctypes.c_int(self.kv_heads), ctypes.c_int(D), ctypes.c_int(cos.shape[0] if cos is not None else 0),
                                     L.ptr(self.k[layer]), L.ptr(self.v[layer]), L.ptr(self.page_table), ctypes.c_int(self.page_size),
                                     ctypes.c_int(self.max_pages), L.stream_ptr()), "rope_append")
        out = torch.empty((R, Hq, D), dtype=qkv.dtype, device=qkv.device)
        sk = getattr(self, "_sinks32", None)
        if sinks is not None and (sk is None or sk[0] is not sinks):
            self._sinks32 = sk = (sinks, sinks.detach().float().contiguous())
        self._fused_decode(lib, layer, qkv, H * D, lens32, R, Hq, D, window, sk[1] if sinks is not None else None, out)
        L.count_launches(1)
        return out

    # ------------------------------------------------------------------ reads
    def gather(self, layer: int, length: int, dtype=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dense ``[R, length, Hkv, D]`` views of the selected rows' first ``length`` cached tokens."""
        R = self.rows if self.row_ids is None else self.row_ids.numel()
        rows = self._rows(R)[:, None].expand(R, length)
        pos = torch.arange(length, device=self.device)[None].expand(R, length)
        slots = self._slots(rows.reshape(-1), pos.reshape(-1))
        kp = self.k[layer].reshape(-1, self.kv_heads, self.head_dim)[slots]
        vp = self.v[layer].reshape(-1, self.kv_heads, self.head_dim)[slots]
        dt = dtype or self.dtype
        if self.kind:
            kp = dequantize(kp, self.k_scale[layer].reshape(-1, self.kv_heads)[slots], dt)
            vp = dequantize(vp, self.v_scale[layer].reshape(-1, self.kv_heads)[slots], dt)
        shape = (R, length, self.kv_heads, self.head_dim)
        return kp.reshape(shape).to(dt), vp.reshape(shape).to(dt)

    def decode_attention(self, layer: int, q: torch.Tensor, lengths: torch.Tensor, scale=None, window=None, sinks=None,
                         softcap: float = 0.0) -> torch.Tensor:
        """``q [R, Hq, D]`` against each row's first ``lengths[r]`` cached tokens -> ``[R, Hq, D]``."""
        R, Hq, D = q.shape
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        if (L.use_cuda(q) and q.dtype == torch.bfloat16 and self.row_ids is None and R == self.rows and not softcap
                and Hq // self.kv_heads <= 8 and D in (64, 128, 256)):
            lib = L.load()
            splits = 1
            longest = self.max_len
            while splits < 16 and R * self.kv_heads * splits < 592 and longest // (splits * 2) >= 256:
                splits *= 2
            # a warp walks its keys 32 at a time with a few dependent memory round trips per step: keep a CTA's share of
            # the longest possible row near 512 keys so that the walk is short and there are CTAs to overlap
            splits = max(splits, min(16, (longest + 511) // 512))
            n = R * Hq * splits
            if self._scratch is None or self._scratch[0].numel() < n:
                self._scratch = (torch.empty(n, dtype=torch.float32, device=q.device), torch.empty(n, dtype=torch.float32, device=q.device),
                                 torch.empty(n * D, dtype=torch.float32, device=q.device))
            pm, pl, pa = self._scratch
            out = torch.empty_like(q)
            qc, lens32 = q.contiguous(), lengths.to(torch.int32).contiguous()      # kept referenced across the launches below
            sinks32 = sinks.float().contiguous() if sinks is not None else None
            if (self.kind == 0 and D == 128 and self.page_size % 64 == 0 and hasattr(lib, "dewb_paged_decode_stream")
                    and os.environ.get("DEWB_DECODE", "stream") == "stream"):
                if scale == 1.0 / math.sqrt(D) and os.environ.get("DEWB_DECODE_FUSED", "1") == "1":
                    self._fused_decode(lib, layer, qc, 0, lens32, R, Hq, D, window, sinks32, out)
                    return out
                # streamed form: TMA page tiles into a shared-memory ring, scores and values on the warp-level tensor cores
                L.check(lib.dewb_paged_decode_stream(L.ptr(qc), L.ptr(self.k[layer]), L.ptr(self.v[layer]),
                                                     ctypes.c_longlong(self.pages * self.page_size), L.ptr(self.page_table), L.ptr(lens32),
                                                     L.ptr(pm), L.ptr(pl), L.ptr(pa), ctypes.c_int(R), ctypes.c_int(Hq),
                                                     ctypes.c_int(self.kv_heads), ctypes.c_int(self.page_size), ctypes.c_int(self.max_pages),
                                                     ctypes.c_int(splits), ctypes.c_float(scale), ctypes.c_int(window or 0),
                                                     ctypes.c_longlong(0), L.ptr(L.status(q.device)), L.stream_ptr()), "paged_decode_stream")
                L.check(lib.dewb_decode_combine(L.ptr(pm), L.ptr(pl), L.ptr(pa), L.ptr(sinks32),
                                                L.ptr(out), L.ptr(None), ctypes.c_int(R), ctypes.c_int(Hq), ctypes.c_int(D), ctypes.c_int(splits),
                                                L.stream_ptr()), "decode_combine")
                L.count_launches(2)
                return out
            L.check(lib.dewb_paged_decode(L.ptr(qc), L.ptr(self.k[layer]), L.ptr(self.v[layer]),
                                          L.ptr(self.k_scale[layer] if self.kind else None),
                                          L.ptr(self.v_scale[layer] if self.kind else None), L.ptr(self.page_table),
                                          L.ptr(lens32), L.ptr(sinks32), L.ptr(out), L.ptr(None),
                                          L.ptr(pm), L.ptr(pl), L.ptr(pa), ctypes.c_int(R), ctypes.c_int(Hq),
                                          ctypes.c_int(self.kv_heads), ctypes.c_int(D), ctypes.c_int(self.page_size),
                                          ctypes.c_int(self.max_pages), ctypes.c_int(splits), ctypes.c_float(scale),
                                          ctypes.c_int(window or 0), ctypes.c_int(self.kind), L.stream_ptr()), "paged_decode")
            L.count_launches(2)
            return out
        return paged_attention_reference(self, layer, q, lengths, scale, window, sinks, softcap)

    # ------------------------------------------------------------------ the call attention layers make
    def attend(self, layer: int, q, k, v, positions, causal=True, window=None, softcap=0.0, sinks=None):
        """Write this call's keys / values, then attend. ``q [R, S, Hq, D]``, ``k, v [R, S, Hkv, D]``, ``positions [R, S]``
        (absolute; -1 marks padding). S == 1 is the decode step (paged kernel); S > 1 is a prefill chunk."""
        R, S = q.shape[0], q.shape[1]
        if positions is None:
            positions = torch.arange(S, device=q.device)[None].expand(R, S)
        if S == 1:
            pos = positions[:, 0]
            self.append(layer, k[:, 0], v[:, 0], pos)
            lengths = torch.where(pos >= 0, pos + 1, torch.zeros_like(pos))
            return self.decode_attention(layer, q[:, 0], lengths, window=window, sinks=sinks, softcap=softcap)[:, None]

        self.write(layer, k, v, positions)
        if self.chunk_span is not None:
            # the caller knows where this chunk starts and ends (a server batching rows by start offset): no device read
            start, total, fresh = self.chunk_span[0], self.chunk_span[1], self.chunk_span[0] == 0
        else:
            start = int(positions[:, 0].clamp_min(0).min())
            fresh = start == 0 and bool((positions[:, 0] <= 0).all())
            total = None
        if fresh:
            return ops.attention(q, k, v, causal=causal, window=window, softcap=softcap, sinks=sinks)
        if total is None:
            total = int(positions.max()) + 1
        kc, vc = self.gather(layer, total, dtype=q.dtype)
        # bottom-right aligned causal attention of the chunk against everything cached so far (rows share `start`)
        return ops.attention_reference(q, kc, vc, causal=causal, window=window, softcap=softcap, sinks=sinks)


def paged_attention_reference(store: KVStore, layer: int, q, lengths, scale, window=None, sinks=None, softcap=0.0):
    """fp32 oracle of the paged decode kernel."""
    R, Hq, D = q.shape
    Lmax = max(int(lengths.max()), 1)
    kc, vc = store.gather(layer, Lmax, dtype=torch.float32)
    rep = Hq // store.kv_heads
    kc, vc = kc.repeat_interleave(rep, 2), vc.repeat_interleave(rep, 2)
    s = torch.einsum("rhd,rthd->rht", q.float(), kc) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    t = torch.arange(Lmax, device=q.device)[None, None]
    mask = t < lengths[:, None, None]
    if window:
        mask = mask & (t >= (lengths[:, None, None] - window))
    s = s.masked_fill(~mask, float("-inf"))
    if sinks is not None:
        p = torch.softmax(torch.cat([s, sinks.float().reshape(1, Hq, 1).expand(R, Hq, 1)], -1), -1)[..., :-1]
    else:
        p = torch.softmax(s, -1)
    p = torch.nan_to_num(p)
    return torch.einsum("rht,rthd->rhd", p, vc).to(q.dtype)
