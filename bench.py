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
    ap.add_argument("--rows", type=int, default=ROWS_PER_GPU, help="sequences per GPU per step")
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (the result is then not a valid headline)")
    ap.add_argument("--skip-e2e", action="store_true")
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

    cfg = dict(MODEL)
    if args.layers:
        cfg["num_layers"] = args.layers
    micro = args.micro or (2 if world == 1 else 4)
    rows = args.rows
    assert rows % micro == 0
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
            "metric": "train tokens/sec (dense 8B LM, FSDP)", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": value / (BASELINE_TOK_S_PER_GPU * world), "dtype": "bf16",
            "data": "synthetic (uniform random token ids from a seed; random-init weights)",
            "config": {"model": "llama-style 8B: d4096 L32 H32/8kv ffn14336 vocab128256", "params": n_params,
                       "global_batch": rows * world, "seq_len": SEQ_LEN, "micro_batch": micro,
                       "parallelism": f"fsdp{world}", "optimizer": "AdamW fp32 masters+moments",
                       "l2": "inputs larger than L2 (16 GB of weights stream every microbatch)",
                       "baseline": "BASELINE.md reference-equivalent mark 190K tok/s at 8xB200, scaled per GPU"},
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
