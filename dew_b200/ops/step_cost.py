"""A cost model of whole steps - a training step under a parallel layout (FSDP / tensor / expert parallel), a decode step under
tensor parallelism - built from single-operation rooflines and collective costs: what a configuration should cost before it is
run, to size a run, to choose a layout, and to read a measurement against.  (``ops.cost`` holds the per-call estimates the
kernel benchmarks print beside their measurements; this module adds collectives, layouts, mixtures, memory and serving.)

Every estimate is a roofline - ``max(FLOPs / tensor throughput, bytes / memory bandwidth)`` - corrected by what the rooflines
leave out: tile quantisation over 148 SMs (a product whose tile count is not a multiple of the SM count runs a partly empty
last wave), a per-launch floor, an efficiency per kernel family taken from this library's measured tables, and for collectives
a latency term plus bytes over the measured NVLink bus bandwidth.  ``Machine.measured()`` reads the peaks measured on the
device pool (``MEASURED_PEAKS.json`` at the repository root when present), else nominal figures.

``gemm_ms`` / ``attention_ms`` / ``rowwise_ms`` / ``collective_ms``   single operations
``transformer_step``   a decoder-only LM's training step on one GPU of a data-parallel / FSDP / TP / EP layout: per-family
                       breakdown, predicted ms, tokens / s, MFU, and the memory the engine's state takes
``decode_step``        a serving step of ``rows`` sequences at a context length under tensor parallelism

Reference: the reference's launch / resource model and roofline constants (src/dew/nn/kernels/generation.py:901-929,
src/dew/nn/kernels/launches.py, src/dew/training/memory.py:69-100).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

SMS = 148


@dataclass(frozen=True)
class Machine:
    bf16_tflops: float = 1414.9          # sustained dense bf16 tensor throughput (a seconds-long loop under the power cap)
    fp8_tflops: float = 2600.0
    hbm_gbs: float = 6553.0
    nvlink_bus_gbs: float = 725.0        # all-reduce bus bandwidth at 8 ranks, large messages
    nvlink_peer_gbs: float = 770.0       # one direction, one peer
    launch_us: float = 2.0               # a launch's floor inside a stream of launches
    collective_latency_us: float = 12.0
    memory_gb: float = 180.0
    source: str = "nominal"

    @classmethod
    def measured(cls, path: Optional[str] = None) -> "Machine":
        path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
        try:
            with open(path) as f:
                rec = json.load(f)
        except (OSError, ValueError):
            return cls()
        return cls(bf16_tflops=float(rec.get("bf16_tflops_sustained", cls.bf16_tflops)), hbm_gbs=float(rec.get("hbm_gbs", cls.hbm_gbs)),
                   fp8_tflops=float(rec.get("bf16_tflops_sustained", cls.bf16_tflops)) * 1.85, source=f"measured {rec.get('when', '')}".strip())


# measured efficiencies of this library's kernels against the rooflines above (fraction of the roofline rate reached on
# large shapes; the tables they come from: the layer-shape GEMM table, the flash-attention table, the row-kernel summaries)
EFFICIENCY = {"gemm": 0.86, "gemm_wgrad": 0.80, "gemm_mx": 0.60, "gemm_grouped": 0.60, "attention_fwd": 0.55, "attention_bwd": 0.50,
              "rowwise": 0.85, "decode_attention": 0.70, "adamw": 0.85, "exchange": 0.45}
# (grouped products over a rank's experts run ragged 128-row tiles and reach less of the peak than one large product; the
# token exchange moves rows in 4 KB pieces and reaches under half of a peer copy's bandwidth: both from the expert-parallel
# step's measured kernel shares)
ACTIVATION_UNITS = 6.5      # saved activations per layer, in units of [tokens, features] bf16 (the gated MLP's wide tensors are recomputed)


def _waves(tiles: int, sms: int = SMS) -> float:
    """The last-wave penalty: time is in whole waves, work only in ``tiles``."""
    return math.ceil(tiles / sms) * sms / max(1, tiles)


def gemm_ms(M: int, N: int, K: int, machine: Machine = Machine(), *, dtype_bytes: int = 2, out_bytes: int = 2, kind: str = "gemm",
            tile=(256, 128)) -> float:
    flops = 2.0 * M * N * K
    bytes_ = dtype_bytes * (M * K + N * K) + out_bytes * M * N
    rate = (machine.fp8_tflops if kind == "gemm_mx" else machine.bf16_tflops) * 1e12 * EFFICIENCY[kind]
    if kind in ("gemm_mx", "gemm_grouped"):
        tile = (128, 192)
    tiles = math.ceil(M / tile[0]) * math.ceil(N / tile[1])
    if tiles < SMS:                                                        # few tiles: the reduction is split over idle SMs
        tiles *= max(1, min(SMS // tiles, K // 512))
    compute = flops / rate * _waves(tiles)
    memory = bytes_ / (machine.hbm_gbs * 1e9 * EFFICIENCY["rowwise"])
    return max(compute, memory) * 1e3 + machine.launch_us * 1e-3


def attention_ms(B: int, S: int, Hq: int, Hkv: int, D: int, machine: Machine = Machine(), *, causal: bool = True, backward: bool = False,
                 window: Optional[int] = None) -> float:
    span = min(S, window) if window else S
    pairs = B * Hq * S * span * (0.5 if causal and not window else 1.0)
    flops = 4.0 * pairs * D * (2.5 if backward else 1.0)            # backward: five products against the forward's two
    rate = machine.bf16_tflops * 1e12 * EFFICIENCY["attention_bwd" if backward else "attention_fwd"]
    bytes_ = 2 * B * S * D * (Hq * 2 + Hkv * 2) * (2.5 if backward else 1.0)
    return max(flops / rate, bytes_ / (machine.hbm_gbs * 1e9)) * 1e3 + machine.launch_us * 1e-3 * (3 if backward else 1)


def rowwise_ms(bytes_moved: float, machine: Machine = Machine(), launches: int = 1) -> float:
    return bytes_moved / (machine.hbm_gbs * 1e9 * EFFICIENCY["rowwise"]) * 1e3 + launches * machine.launch_us * 1e-3


def collective_ms(kind: str, bytes_per_rank: float, world: int, machine: Machine = Machine()) -> float:
    """``bytes_per_rank``: the full tensor's size for all_reduce / all_gather (the gathered size) / reduce_scatter (the input size);
    the bytes a rank sends for all_to_all."""
    if world <= 1:
        return 0.0
    lat = machine.collective_latency_us * 1e-3
    if kind == "all_reduce":
        return lat + 2 * (world - 1) / world * bytes_per_rank / (machine.nvlink_bus_gbs * 1e9) * 1e3
    if kind in ("all_gather", "reduce_scatter"):
        return lat + (world - 1) / world * bytes_per_rank / (machine.nvlink_bus_gbs * 1e9) * 1e3
    if kind == "all_to_all":
        return lat + (world - 1) / world * bytes_per_rank / (machine.nvlink_peer_gbs * 1e9) * 1e3
    if kind == "send":
        return lat + bytes_per_rank / (machine.nvlink_peer_gbs * 1e9) * 1e3
    raise ValueError(f"unknown collective {kind!r}")


@dataclass
class Transformer:
    """A decoder-only LM's shape (the dense 8 B flagship by default); ``experts`` > 0 makes every layer's MLP a mixture."""
    features: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    mlp: int = 14336
    vocab: int = 128256
    experts: int = 0
    top_k: int = 0
    expert_mlp: int = 0
    shared_experts: int = 0
    tied: bool = False

    @property
    def layer_params(self) -> float:
        attn = self.features * self.head_dim * (self.heads + 2 * self.kv_heads) + self.heads * self.head_dim * self.features
        if self.experts:
            mlp = 3 * self.features * self.expert_mlp * (self.experts + self.shared_experts) + self.features * self.experts
        else:
            mlp = 3 * self.features * self.mlp
        return attn + mlp + 2 * self.features

    @property
    def params(self) -> float:
        return self.layers * self.layer_params + self.vocab * self.features * (1 if self.tied else 2) + self.features

    @property
    def active_layer_params(self) -> float:
        if not self.experts:
            return self.layer_params
        attn = self.features * self.head_dim * (self.heads + 2 * self.kv_heads) + self.heads * self.head_dim * self.features
        return attn + 3 * self.features * self.expert_mlp * (self.top_k + self.shared_experts) + self.features * self.experts


def transformer_step(model: Transformer, *, sequences: int, seq_len: int, microbatch: int = 4, world: int = 1, tensor: int = 1, expert: int = 1,
                     machine: Optional[Machine] = None, remat: bool = False, mx_experts: bool = False, sharded_state: bool = False) -> Dict[str, Any]:
    """One GPU's training step: ``sequences`` of ``seq_len`` tokens on this GPU in microbatches of ``microbatch`` sequences, FSDP over
    ``world // tensor`` ranks, tensor parallel over ``tensor``, expert parallel over ``expert``.  Returns the per-family milliseconds,
    the step's total, tokens / s for the whole job, MFU against the datasheet and against the measured peak, and state memory."""
    m = machine or Machine.measured()
    tokens_mb = microbatch * seq_len
    n_mb = max(1, sequences // microbatch)
    d, hd = model.features, model.head_dim
    hq, hkv = model.heads // tensor, max(1, model.kv_heads // tensor)
    fam: Dict[str, float] = {}

    def add(name, ms):
        fam[name] = fam.get(name, 0.0) + ms

    def linear(name, n_out, n_in, rows=tokens_mb, kind="gemm"):
        # forward, input gradient, weight gradient
        add(name, gemm_ms(rows, n_out, n_in, m, kind=kind) + gemm_ms(rows, n_in, n_out, m, kind=kind)
            + gemm_ms(n_out, n_in, rows, m, kind="gemm_wgrad", out_bytes=4))

    per_layer_before = dict(fam)
    linear("gemm", (hq + 2 * hkv) * hd, d)
    linear("gemm", d, hq * hd)
    if model.experts:
        rows = tokens_mb * model.top_k                                     # routed rows, balanced over the experts of this rank
        kind = "gemm_mx" if mx_experts else "gemm_grouped"
        linear("expert_gemm", 2 * model.expert_mlp, d, rows, kind)
        linear("expert_gemm", d, model.expert_mlp, rows, kind)
        if mx_experts:                                                     # quantising the operands: a read and a (half-size) write each
            add("expert_gemm", 6 * rowwise_ms(rows * d * 3, m) + 4 * rowwise_ms(rows * model.expert_mlp * 3 * 1.5, m))
        if model.shared_experts:
            linear("gemm", 2 * model.expert_mlp * model.shared_experts, d)
            linear("gemm", d, model.expert_mlp * model.shared_experts)
        add("gemm", 3 * gemm_ms(tokens_mb, model.experts, d, m))            # the router
        if expert > 1:
            sent = rows * d * 2                                            # dispatch and combine, forward and backward
            # routing (scores, top-k, ranks, the plan: a dozen small launches each way), the four exchanges, the passes over the
            # receive buffer around them (zeroing padding rows, the weighted combine and its backward)
            add("exchange", 4 * collective_ms("all_to_all", sent, expert, m) / EFFICIENCY["exchange"] + 6 * rowwise_ms(2 * sent, m)
                + 48 * m.launch_us * 1e-3 + 4 * m.collective_latency_us * 1e-3)
    else:
        linear("gemm", 2 * model.mlp // tensor, d)
        linear("gemm", d, model.mlp // tensor)
    B = microbatch
    add("attention", attention_ms(B, seq_len, hq, hkv, hd, m) + attention_ms(B, seq_len, hq, hkv, hd, m, backward=True))
    act = tokens_mb * d * 2
    # norms (two per layer, forward + backward), rotary, the gated activation, residual adds
    width = (model.expert_mlp * (model.top_k + model.shared_experts)) if model.experts else model.mlp // tensor
    add("rowwise", 2 * rowwise_ms(3 * act, m) + 2 * rowwise_ms(4 * act, m) + rowwise_ms(tokens_mb * width * 2 * 3, m) + rowwise_ms(tokens_mb * width * 2 * 5, m)
        + 2 * rowwise_ms(tokens_mb * (hq + hkv) * hd * 2 * 2, m))
    if tensor > 1:
        add("tensor_parallel", 4 * collective_ms("all_reduce", act, tensor, m))
    if remat:
        extra = {k: v - per_layer_before.get(k, 0.0) for k, v in fam.items()}
        for k, v in extra.items():
            fam[k] += v / 3.0                                              # the forward third is run again in the backward
    for k in list(fam):
        fam[k] *= model.layers * n_mb
    # the head: a chunked cross-entropy (logits never stored) = three products over the vocabulary
    rows_all = n_mb * tokens_mb
    fam["head"] = n_mb * (gemm_ms(tokens_mb, model.vocab // tensor, d, m) * 2 + gemm_ms(model.vocab // tensor, d, tokens_mb, m, kind="gemm_wgrad", out_bytes=4)
                          + rowwise_ms(tokens_mb * (model.vocab // tensor) * 2 * 2, m, 2))
    # the update: reduce-scatter of fp32 gradients, AdamW on the shard, all-gather of bf16 parameters - once per step
    fsdp = max(1, world // tensor)
    local = model.params / tensor
    if model.experts and expert > 1:
        expert_params = model.layers * 3 * d * model.expert_mlp * model.experts
        local = (model.params - expert_params) + expert_params / expert
    fam["update"] = rowwise_ms(local / fsdp * (4 * 3 * 2 + 4 + 2), m) + collective_ms("reduce_scatter", local * 4, fsdp, m) \
        + collective_ms("all_gather", local * 2, fsdp, m)
    if sharded_state and fsdp > 1:
        fam["gather"] = n_mb * 2 * collective_ms("all_gather", local * 2, fsdp, m) * 0.15          # mostly hidden behind the products
    total = sum(fam.values())
    tokens = rows_all * world / tensor
    step_flops = 6.0 * (model.layers * model.active_layer_params + model.vocab * d) * rows_all \
        + 12.0 * model.layers * n_mb * B * model.heads / tensor * seq_len * seq_len * hd * 0.5 * (1 + 1.0)
    state = {"bf16_weights": local * 2 / (fsdp if sharded_state else 1), "fp32_gradients": local * 4 / (fsdp if sharded_state else 1),
             "optimizer": local * 12 / fsdp}
    acts = tokens_mb * d * 2 * model.layers * (2 if remat else ACTIVATION_UNITS)
    return {"ms": total, "by_family": fam, "tokens_per_s": tokens / (total * 1e-3), "tokens_per_s_per_gpu": rows_all / tensor / (total * 1e-3),
            "mfu_datasheet": step_flops / (total * 1e-3) / 2.25e15, "mfu_measured": step_flops / (total * 1e-3) / (m.bf16_tflops * 1e12),
            "state_gb": {k: v / 1e9 for k, v in state.items()}, "activation_gb": acts / 1e9,
            "memory_gb": (sum(state.values()) + acts) / 1e9, "fits": (sum(state.values()) + acts) / 1e9 < m.memory_gb * 0.92, "machine": m.source}


def decode_step(model: Transformer, *, rows: int, context: int, tensor: int = 1, machine: Optional[Machine] = None, kv_bytes: int = 2) -> Dict[str, Any]:
    """One decode step of ``rows`` sequences, each attending over ``context`` cached tokens, under ``tensor``-way tensor parallelism:
    the weights are read once (``rows`` is small, the products are bandwidth-bound), the cache once, and every layer pays two
    small all-reduces."""
    m = machine or Machine.measured()
    d, hd = model.features, model.head_dim
    weights = model.layers * model.active_layer_params * 2 / tensor
    fam = {"weights": rowwise_ms(weights, m, launches=4 * model.layers),
           "kv_cache": model.layers * (2 * rows * context * max(1, model.kv_heads // tensor) * hd * kv_bytes) / (m.hbm_gbs * 1e9 * EFFICIENCY["decode_attention"]) * 1e3
           + model.layers * m.launch_us * 1e-3,
           "head": rowwise_ms(model.vocab * d * 2 / tensor, m, 2),
           "rowwise": model.layers * 4 * m.launch_us * 1e-3}
    if tensor > 1:
        fam["all_reduce"] = model.layers * 2 * (m.collective_latency_us * 1e-3 + collective_ms("all_reduce", rows * d * 2, tensor, m) - m.collective_latency_us * 1e-3)
        fam["all_reduce"] += model.layers * 2 * m.collective_latency_us * 1e-3
    total = sum(fam.values())
    return {"ms": total, "by_family": fam, "tokens_per_s": rows / (total * 1e-3), "machine": m.source}


PRESETS = {
    "dense8b": Transformer(),
    "moe": Transformer(features=2048, layers=24, heads=16, kv_heads=16, head_dim=128, mlp=0, vocab=32768, experts=64, top_k=6, expert_mlp=1408, shared_experts=2),
    "qwen3_0p6b": Transformer(features=1024, layers=28, heads=16, kv_heads=8, head_dim=128, mlp=3072, vocab=151936, tied=True),
    "llama70b": Transformer(features=8192, layers=80, heads=64, kv_heads=8, head_dim=128, mlp=28672, vocab=128256),
}


def main(argv=None) -> Dict[str, Any]:
    import argparse
    ap = argparse.ArgumentParser(description="Predict a training or decode step's cost on B200s.")
    ap.add_argument("--model", default="dense8b", choices=sorted(PRESETS))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--tensor", type=int, default=1)
    ap.add_argument("--expert", type=int, default=1)
    ap.add_argument("--sequences", type=int, default=32, help="sequences per GPU per step")
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--microbatch", type=int, default=4)
    ap.add_argument("--remat", action="store_true")
    ap.add_argument("--sharded", action="store_true")
    ap.add_argument("--decode", type=int, default=0, help="predict a decode step of this many rows instead")
    ap.add_argument("--context", type=int, default=2048)
    args = ap.parse_args(argv)
    model = PRESETS[args.model]
    if args.decode:
        out = decode_step(model, rows=args.decode, context=args.context, tensor=args.tensor)
    else:
        out = transformer_step(model, sequences=args.sequences, seq_len=args.seq_len, microbatch=args.microbatch, world=args.gpus, tensor=args.tensor,
                               expert=args.expert, remat=args.remat, sharded_state=args.sharded, mx_experts=bool(model.experts))
    print(json.dumps(out, indent=1, default=float))
    return out


if __name__ == "__main__":
    main()
