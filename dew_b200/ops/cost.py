"""A roofline cost model for the library's ops: the time a call should take on this GPU, from its FLOPs and bytes, the
measured peaks of the device and a measured efficiency per kernel family.

Used to rank candidate plans before anything runs (microbatch sizes in ``training.planning``, engine choice), to print the
expected time beside a measured one in the kernel benchmarks, and by tests that pin the model's arithmetic.  The peaks come
from ``MEASURED_PEAKS.json`` when present (copy bandwidth, cuBLAS bf16 burst / sustained) and from this pool's recorded
fallback otherwise; the efficiencies are the fractions of those peaks the kernels reached in the committed profiles.

Reference: the kernel cost model of src/dew/nn/kernels/generation.py:901-929 (device facts) and the launch / resource model
of src/dew/nn/kernels/launches.py.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Optional


@dataclass(frozen=True)
class Device:
    hbm_gbs: float = 6650.0            # STREAM-style copy bandwidth
    bf16_tflops: float = 1590.0        # cuBLAS burst
    bf16_tflops_sustained: float = 1400.0
    fp8_ratio: float = 2.0             # dense fp8 over bf16 tensor throughput
    nvlink_gbs: float = 770.0          # peer copy, per direction
    launch_us: float = 2.5             # back-to-back launch cost inside a stream
    sms: int = 148
    source: str = "fallback"


def device() -> Device:
    here = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    path = os.environ.get("DEWB_MEASURED_PEAKS", str(here))
    try:
        with open(path) as f:
            m = json.load(f)
        return Device(hbm_gbs=float(m["hbm_gbs"]), bf16_tflops=float(m["bf16_tflops"]),
                      bf16_tflops_sustained=float(m.get("bf16_tflops_sustained", m["bf16_tflops"])), source="measured")
    except (OSError, KeyError, ValueError):
        return Device()


# fraction of the matching peak each kernel family reaches (from the committed profiles)
EFFICIENCY: Dict[str, float] = {
    "gemm_pair": 0.86, "gemm_single": 0.80, "gemm_mx": 0.70, "grouped_gemm": 0.70, "flash_fwd": 0.42, "flash_bwd": 0.40,
    "rows": 0.90, "paged_decode": 0.55, "gdn": 0.30, "ssd": 0.30, "peer_copy": 0.85,
}


@dataclass(frozen=True)
class Estimate:
    ms: float
    bound: str                 # "compute" | "memory" | "link" | "launch"
    compute_ms: float
    memory_ms: float
    link_ms: float = 0.0


def estimate(flops: float, bytes_moved: float, kernel: str = "gemm_pair", dev: Optional[Device] = None, fp8: bool = False,
             link_bytes: float = 0.0, launches: int = 1, sustained: bool = False) -> Estimate:
    """Time of one call: the slowest of FLOPs over tensor peak, bytes over copy bandwidth and peer bytes over the link, each
    divided by the kernel family's efficiency, and never below the launch cost."""
    dev = dev or device()
    eff = EFFICIENCY.get(kernel, 0.7)
    peak = (dev.bf16_tflops_sustained if sustained else dev.bf16_tflops) * (dev.fp8_ratio if fp8 else 1.0)
    c = flops / (peak * 1e12 * eff) * 1e3 if flops else 0.0
    m = bytes_moved / (dev.hbm_gbs * 1e9 * EFFICIENCY.get("rows", 0.9)) * 1e3 if bytes_moved else 0.0
    l = link_bytes / (dev.nvlink_gbs * 1e9 * EFFICIENCY.get("peer_copy", 0.85)) * 1e3 if link_bytes else 0.0
    floor = launches * dev.launch_us * 1e-3
    t = max(c, m, l, floor)
    bound = "launch" if t == floor and floor > max(c, m, l) else ("compute" if t == c else "memory" if t == m else "link")
    return Estimate(t, bound, c, m, l)


def gemm(M: int, N: int, K: int, out_bytes: int = 2, kernel: str = "gemm_pair", **kw) -> Estimate:
    return estimate(2.0 * M * N * K, 2.0 * (M * K + N * K) + out_bytes * M * N, kernel, **kw)


def attention(B: int, S: int, Hq: int, Hkv: int, D: int, causal: bool = True, backward: bool = False, **kw) -> Estimate:
    pairs = S * (S + 1) / 2 if causal else S * S
    flops = 4.0 * B * Hq * pairs * D * (2.5 if backward else 1.0)
    bytes_moved = 2.0 * B * S * D * (2 * Hq + 2 * Hkv) * (2 if backward else 1)
    return estimate(flops, bytes_moved, "flash_bwd" if backward else "flash_fwd", **kw)


def decoder_step(tokens: int, d: int, layers: int, ffn: int, heads: int, kv_heads: int, head_dim: int, vocab: int, seq: int,
                 dev: Optional[Device] = None) -> Dict[str, float]:
    """Forward + backward time of one microbatch of a dense decoder, by kernel family (ms), and the total."""
    qkv = (heads + 2 * kv_heads) * head_dim
    per_layer = [gemm(tokens, qkv, d, dev=dev, sustained=True), gemm(tokens, d, heads * head_dim, dev=dev, sustained=True),
                 gemm(tokens, 2 * ffn, d, dev=dev, sustained=True), gemm(tokens, d, ffn, dev=dev, sustained=True)]
    gemm_ms = 3.0 * sum(e.ms for e in per_layer) * layers + 3.0 * gemm(tokens, vocab, d, dev=dev, sustained=True).ms
    B = max(1, tokens // seq)
    attn_ms = layers * (attention(B, seq, heads, kv_heads, head_dim, dev=dev).ms + attention(B, seq, heads, kv_heads, head_dim, backward=True, dev=dev).ms)
    rows_bytes = tokens * (d * 2 * 14 + ffn * 2 * 5)
    rows_ms = layers * estimate(0.0, rows_bytes, "rows", dev=dev).ms
    return {"gemm_ms": gemm_ms, "attention_ms": attn_ms, "rows_ms": rows_ms, "total_ms": gemm_ms + attn_ms + rows_ms}
