"""Headline benchmark: training tokens per second of the dense Llama-style 8 B decoder (d_model 4096, 32 layers,
32 query / 8 KV heads, SwiGLU 14336, vocab 128256, sequence 4096, AdamW, bf16 compute with fp32 masters) under FSDP
on N GPUs of one node, weak scaling at 32 sequences per GPU per step (256 sequences at 8 GPUs).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 5 --warmup 3

Prints ONE JSON line (rank 0).  ``value`` is device-timed (CUDA events, barrier + synchronize on both sides, max over
ranks) with inputs already on the device; ``e2e`` is the same metric through ``Trainer.fit`` with each step's tokens
copied from pinned host memory and the step's loss read back to the host.  Data is synthetic (token ids uniform
over the vocabulary from a seed) and weights are random-init.  ``--impl reference`` reports on the reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")

BASELINE_TOK_S_PER_GPU = 190_000 / 8      # reference-equivalent mark for this config (8 x B200), per GPU

MODEL = dict(vocab_size=128256, emb_features=4096, num_layers=32, num_heads=32, num_kv_heads=8, head_dim=128,
             mlp_features=14336, max_seq_len=4096, rope_theta=500000.0, qk_norm=False, tie_embeddings=False,
             norm_eps=1e-5)
SEQ_LEN = 4096
ROWS_PER_GPU = 32

# The other training configurations (selected with --config; the headline above is the default and the only one the
# one-line contract of this script describes):
#   moe     d_model 2048, 24 layers, 16 heads, 64 routed experts (FFN 1408, SwiGLU) top-6 softmax + 2 shared experts,
#           row-scaled fp8 expert GEMMs, expert parallelism over all N ranks, sequence 4096, 16 sequences per GPU
#   hybrid  d_model 2048, 24 layers in a 3 x gated-delta-net (16 heads x 128, short conv 4) + 1 x attention pattern,
#           sequence 8192, 8 sequences per GPU, FSDP
CONFIGS = {
    "dense": dict(model=MODEL, seq=4096, rows=32, metric="train tokens/sec (dense 8B LM, FSDP)",
                  name="llama-style 8B: d4096 L32 H32/8kv ffn14336 vocab128256"),
    "moe": dict(model=dict(vocab_size=32768, emb_features=2048, num_layers=24, num_heads=16, num_kv_heads=16, head_dim=128,
                           mlp_features=1408, max_seq_len=4096, qk_norm=False, tie_embeddings=False, norm_eps=1e-5),
                mixture=dict(experts=64, top_k=6, expert_features=1408, shared_features=2 * 1408, fp8=True),
                seq=4096, rows=16, metric="train tokens/sec (MoE LM, expert parallel)",
                name="MoE: d2048 L24 H16 64 experts x 1408 top-6 + 2 shared, fp8 expert GEMMs, vocab 32768"),
    "hybrid": dict(model=dict(vocab_size=32768, emb_features=2048, num_layers=24, num_heads=16, num_kv_heads=16, head_dim=128,
                              mlp_features=5632, max_seq_len=8192, qk_norm=False, tie_embeddings=False, norm_eps=1e-5,
                              layer_types=("gdn", "gdn", "gdn", "attention"),
                              mixer_options=dict(num_k_heads=16, num_v_heads=16, head_k_dim=128, head_v_dim=128, conv_size=4)),
                   seq=8192, rows=8, metric="train tokens/sec (hybrid GDN LM, FSDP)",
                   name="hybrid: d2048 L24 (3 gated-delta-net 16x128 conv4 : 1 attention), vocab 32768"),
}


def reference_arm(args) -> None:
    """The reference needs its pinned JAX fork (jax 0.12.0.1.post118 + jaxlib / PJRT plugin) and flax / optax /
    orbax, none of which exist offline; `pip install --no-deps` installs the package but `import dew` fails."""
    reason = "reference installs only with --no-deps; `import dew` fails: No module named 'jax' (pinned JAX fork, flax, optax, orbax not available offline)"
    try:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref"))
        import dew  # noqa: F401
        reason = "reference imported but its JAX CUDA plugin for sm_100 (cuda13 build) is not installed"
    except Exception as e:  # the expected outcome on this image
        reason = f"reference cannot be imported: {type(e).__name__}: {str(e)[:120]}"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason}))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, f"/tmp/dewb_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        # samples under load: the upper half of the clock samples excludes idle gaps between phases
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="dew_b200")
    ap.add_argument("--micro", type=int, default=None, help="sequences per microbatch (default 2 at N=1, where memory allows no more, 4 otherwise)")
    ap.add_argument("--rows", type=int, default=None, help="sequences per GPU per step (default: the configuration's)")
    ap.add_argument("--config", default="dense", choices=sorted(CONFIGS), help="training configuration (default: the headline)")
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (the result is then not a valid headline)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"],
                    help="moe: token exchange by this library's peer-memory kernels (default) or by NCCL all-to-all (comparison arm)")
    ap.add_argument("--profile", default=None, help="write a torch.profiler kernel table for one step to this file")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    import dew_b200 as dew
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective
    from dew_b200.ops import library as L
    from dew_b200.parallel.fsdp import FSDPEngine

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L.load()

    conf = CONFIGS[args.config]
    SEQ_LEN = conf["seq"]
    cfg = dict(conf["model"])
    if args.layers:
        cfg["num_layers"] = args.layers
    micro = args.micro or ((2 if world == 1 else 4) if args.config == "dense" else 2)
    rows = args.rows or conf["rows"]
    assert rows % micro == 0
    if args.config == "moe":
        # experts are split over the ranks before the engine takes the parameters: build on the device, same seed everywhere
        from dew_b200.models.causal_transformer import Mixture
        from dew_b200.nn.layers import reset_all
        from dew_b200.parallel.ep import ExpertParallel
        model = CausalTransformer(device=dev, dtype=torch.bfloat16, mixture=Mixture(**conf["mixture"]), **cfg)
        reset_all(model, 1234)
        if world > 1:
            ExpertParallel(fused=args.ep == "peer").shard(model)
        else:
            next(p for n, p in model.named_parameters() if "experts.gate_up" in n).expert_parallel = True   # initialised above
        torch.cuda.empty_cache()
    else:
        model = CausalTransformer(device="meta", dtype=torch.bfloat16, **cfg)
    objective = LMObjective(model, SEQ_LEN, ema_decay=None)
    tracker = dew.MemoryTracker()
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=3e-4, weight_decay=0.1, optimizer_opts={"b2": 0.95}),
                          key=0, microbatches=rows // micro, param_dtype=torch.bfloat16, tracker=tracker)
    trainer.device = dev
    engine = FSDPEngine(trainer)
    trainer._engine = engine
    state = engine.fresh_state(trainer.key)
    n_params = sum(p.numel() for p in model.parameters())

    gen = torch.Generator().manual_seed(1234 + rank)
    n_batches = args.warmup + 2 * args.steps + 2
    host = [torch.randint(0, cfg["vocab_size"], (rows, SEQ_LEN + 1), generator=gen).pin_memory() for _ in range(n_batches)]
    device_batches = [{"tokens": h.to(dev)} for h in host[: args.warmup + args.steps]]

    def sync():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-timed region (inputs resident)
    for i in range(args.warmup):
        try:
            state, metrics = engine.step(state, device_batches[i])
        except torch.cuda.OutOfMemoryError:
            # one GPU holds all 144 GB of parameter / optimizer state; if the allocator cannot fit two sequences of
            # activations beside it, fall back to one sequence per microbatch (decided in the untimed warm-up only)
            if world > 1 or micro == 1:
                raise
            micro = 1
            trainer.microbatches = rows
            for p in model.parameters():
                p.grad = None
            torch.cuda.empty_cache()
            state, metrics = engine.step(state, device_batches[i])
    sync()
    L.check_status()
    if args.profile:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            state, metrics = engine.step(state, device_batches[0])
            torch.cuda.synchronize(dev)
        if rank == 0:
            with open(args.profile, "w") as f:
                f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=60, max_name_column_width=90))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.LAUNCHES
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    start.record()
    for i in range(args.steps):
        state, metrics = engine.step(state, device_batches[args.warmup + i])
    end.record()
    sync()
    ms = start.elapsed_time(end)
    launches = L.LAUNCHES - launches0
    clocks = sampler.stop() if rank == 0 else None
    L.check_status()
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    loss = float(metrics["loss"].value())
    tokens_per_step = rows * SEQ_LEN * world
    value = tokens_per_step * args.steps / (ms / 1e3)

    # ---- end to end through Trainer.fit: pinned host tokens in, loss out, every step
    e2e = None
    if not args.skip_e2e:
        class HostBatches:
            batch, seq_len = rows, SEQ_LEN

            def __iter__(self):
                i = args.warmup + args.steps
                while True:
                    yield {"tokens": host[i % len(host)]}
                    i += 1
        losses = []
        trainer.fit(HostBatches(), state=state, steps=state.step + 1, log_every=1, checkpoint_final=False)   # warm the path
        sync()
        t0 = time.perf_counter()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        state = trainer.fit(HostBatches(), state=state, steps=state.step + args.steps, log_every=1, checkpoint_final=False,
                            observe=lambda st, m: losses.append(float(m["loss"].value())))
        e2.record()
        sync()
        ms2 = s2.elapsed_time(e2)
        if world > 1:
            t = torch.tensor([ms2], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms2 = float(t.item())
        e2e = {"value": tokens_per_step * args.steps / (ms2 / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": rows * (SEQ_LEN + 1) * 8 * world, "d2h_bytes_per_step": 8 * world,
               "ms_per_step": ms2 / args.steps}
        L.check_status()

    if rank == 0:
        flops = model.model_flops(tokens_per_step // world, SEQ_LEN) * 3
        mfu = flops * args.steps / (ms / 1e3) / 2.25e15
        out = {
            "metric": conf["metric"], "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": value / (BASELINE_TOK_S_PER_GPU * world) if args.config == "dense" else None,
            "dtype": "bf16" if args.config != "moe" else "bf16 (fp8 e4m3 expert GEMMs)",
            "data": "synthetic (uniform random token ids from a seed; random-init weights)",
            "config": {"model": conf["name"], "params": n_params,
                       "global_batch": rows * world, "seq_len": SEQ_LEN, "micro_batch": micro,
                       "parallelism": f"fsdp{world}" + (f"+ep{world} ({args.ep} exchange)" if args.config == "moe" else ""),
                       "optimizer": "AdamW fp32 masters+moments",
                       "l2": "inputs larger than L2 (16 GB of weights stream every microbatch)",
                       "baseline": "reference-equivalent mark 190K tok/s at 8xB200, scaled per GPU"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "loss": loss, "mfu_datasheet": mfu,
            "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 1e9, "impl": "dew_b200",
        }
        if args.layers:
            out["invalid"] = "debug run with fewer layers"
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
