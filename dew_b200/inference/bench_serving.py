"""Serving benchmark: continuous batching of concurrent requests on a tensor-parallel decoder.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29501 \\
        -m dew_b200.inference.bench_serving --requests 128 --new-tokens 256

Workload (the reference's matched greedy workload, tools/benchmark_lm_serving.py:1-80, at the target configuration):
the dense 8 B decoder in bf16 with random-init weights, paged KV cache, ``--requests`` concurrent requests with prompt
lengths uniform in [128, 2048] from a seed, ``--new-tokens`` greedy output tokens each.  Reports decode tokens per
second (device-timed over the decode phase, max over ranks) and time-to-first-token percentiles.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import time

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=128)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--prefill-rows", type=int, default=16384, help="rows the fused all-reduce buffers hold (a prefill step's token budget)")
    ap.add_argument("--out", default=None)
    ap.add_argument("--profile", default=None, help="write a torch.profiler kernel table of eight decode steps to this file")
    ap.add_argument("--arrival-rate", type=float, default=0.0,
                    help="open loop: requests arrive as a Poisson process of this many per second (seeded) while the server runs; "
                         "time to first token and inter-token latency are measured from each request's own arrival")
    args = ap.parse_args(argv)

    from ..models import CausalTransformer
    from ..nn.kv_cache import KVCache
    from ..ops import library as L
    from ..parallel.tp import TensorParallel, tensor_parallelize
    from .serving import Server

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    cfg = dict(vocab_size=128256, emb_features=4096, num_layers=args.layers, num_heads=32, num_kv_heads=8, head_dim=128,
               mlp_features=14336, max_seq_len=max(4096, args.max_prompt + args.new_tokens), rope_theta=500000.0, qk_norm=False, tie_embeddings=False, norm_eps=1e-5)
    torch.manual_seed(0)
    # build and shard layer by layer on the device in bf16 (same seed on every rank -> identical full weights)
    model = CausalTransformer(dtype=torch.bfloat16, device=dev, **cfg).eval()
    for p in model.parameters():
        p.requires_grad_(False)
    capacity = args.max_prompt + args.new_tokens
    tp = TensorParallel(None, max_rows=max(args.requests, args.chunk, args.prefill_rows), features=cfg["emb_features"], device=dev)
    tensor_parallelize(model, tp)
    torch.cuda.empty_cache()
    server = Server(model, slots=args.requests, capacity=capacity, kv_cache=KVCache(page_size=args.page_size),
                    chunk=args.chunk, prefix_cache=False, cuda_graph=not args.no_graph)
    g = torch.Generator().manual_seed(1234)
    lens = torch.randint(args.min_prompt, args.max_prompt + 1, (args.requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]

    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if args.arrival_rate > 0:
        return open_loop(args, server, prompts, lens, rank, world, dev, L)
    # a warm server: one short request first (library handles, lazily loaded kernels, the decode graph), outside the measurement
    server.submit(prompts[0][:args.min_prompt], 4)
    server.run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    tickets = [server.submit(p, args.new_tokens) for p in prompts]
    if args.profile:
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA]) as pprof:
            for _ in range(2):
                server.step()
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.profile + ".prefill", "w") as f:
                f.write(pprof.key_averages().table(sort_by="self_cuda_time_total", row_limit=40, max_name_column_width=90))
    # prefill phase: step until every row has its prompt in the cache
    while any(r is None or r.prefilled < len(r.ticket.prompt) for r in server.rows) and server.busy:
        server.step()
    torch.cuda.synchronize()
    t_prefill = time.perf_counter() - t0
    if args.profile:
        for _ in range(3):
            server.step()
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA]) as prof:
            for _ in range(8):
                server.step()
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.profile, "w") as f:
                f.write(prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=40, max_name_column_width=90))
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    decoded0 = server.decoded_tokens
    steps0 = server.steps
    wait0, wall0 = server.wait_s, time.perf_counter()
    start.record()
    server.run()
    end.record()
    torch.cuda.synchronize()
    host_busy_ms = 1e3 * ((time.perf_counter() - wall0) - (server.wait_s - wait0)) / max(1, server.steps - steps0)
    L.check_status()
    ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # the decode step by itself: the captured graph replayed back to back at the final sequence lengths (no host work between
    # replays), so that a step bound by the host shows as a gap between this number and ms_per_decode_step
    graph_ms = None
    if getattr(server, "_graph", None) is not None:
        server._in_pos.copy_(torch.tensor([n + args.new_tokens - 2 for n in lens], device=dev))
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        start.record()
        for _ in range(20):
            server._graph.replay()
        end.record()
        torch.cuda.synchronize()
        L.check_status()
        graph_ms = start.elapsed_time(end) / 20
    new_tokens = sum(len(t.tokens) for t in tickets)
    decode_tokens = server.decoded_tokens - decoded0
    ttft = sorted(t.first_token_time for t in tickets)
    out = {"metric": "TP decode tokens/sec", "value": decode_tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
           "requests": args.requests, "new_tokens_each": args.new_tokens, "decode_steps": server.steps - steps0,
           "ms_per_decode_step": ms / max(1, server.steps - steps0), "graph_replay_ms": graph_ms, "host_busy_ms_per_step": host_busy_ms, "prefill_s": t_prefill,
           "ttft_p50_s": ttft[len(ttft) // 2], "ttft_p90_s": ttft[int(len(ttft) * 0.9)], "total_new_tokens": new_tokens,
           "prompt_tokens": sum(lens), "layers": args.layers, "cuda_graph": not args.no_graph, "page_size": args.page_size,
           "dtype": "bf16", "data": "synthetic prompts, random-init weights", "gpu_launches": L.LAUNCHES}
    if rank == 0:
        print(json.dumps(out))
        if args.out:
            with open(args.out, "a") as f:
                f.write(json.dumps(out) + "\n")
    if world > 1:
        # Leave through a barrier and a hard exit: tearing the NCCL communicator down after its collectives were
        # captured into a CUDA graph can block, and nothing remains to be flushed but stdout.
        dist.barrier()
        torch.cuda.synchronize()
    import sys
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def open_loop(args, server, prompts, lens, rank, world, dev, L):
    """Open-loop workload (the reference's arrival harness, tools/benchmark_lm_serving.py:60-80): request i arrives at a seeded
    Poisson time whether or not the server is busy; rank 0's clock decides how many have arrived before each step and tells
    the other ranks, so that every tensor-parallel rank admits the same requests at the same step."""
    import random
    rng = random.Random(4321)
    at, arrivals = 0.0, []
    for _ in prompts:
        at += rng.expovariate(args.arrival_rate)
        arrivals.append(at)
    # warm the kernels / graphs outside the measurement
    warm = server.submit(prompts[0][:128], 4)
    server.run()
    torch.cuda.synchronize()
    tickets, token_times = [], {}
    nxt = 0
    count = torch.zeros(1, dtype=torch.int64, device=dev)
    t0 = time.perf_counter()
    while nxt < len(prompts) or server.busy:
        now = time.perf_counter() - t0
        due = nxt
        while due < len(prompts) and arrivals[due] <= now:
            due += 1
        if world > 1:
            count[0] = due
            dist.broadcast(count, src=0)
            due = int(count.item())
        for i in range(nxt, due):
            times = []
            t = server.submit(prompts[i], args.new_tokens, on_token=lambda tok, times=times: times.append(time.perf_counter()))
            t.submitted = t0 + arrivals[i]                          # measured from the arrival, not from the admission
            tickets.append(t)
            token_times[id(t)] = times
        nxt = due
        if server.busy:
            server.step()
        else:
            time.sleep(min(0.001, max(0.0, arrivals[nxt] - now))) if nxt < len(prompts) else None
    torch.cuda.synchronize()
    total_s = time.perf_counter() - t0
    L.check_status()
    ttft = sorted(t.first_token_time for t in tickets if t.first_token_time is not None)
    itl = sorted(b - a for t in tickets for a, b in zip(token_times[id(t)], token_times[id(t)][1:]))
    pct = lambda xs, p: xs[min(len(xs) - 1, int(len(xs) * p))] if xs else None
    out = {"metric": "open-loop serving", "arrival_rate_per_s": args.arrival_rate, "requests": len(tickets), "n_gpus": world,
           "new_tokens_each": args.new_tokens, "output_tokens_per_s": sum(len(t.tokens) for t in tickets) / total_s,
           "ttft_p50_s": pct(ttft, 0.5), "ttft_p90_s": pct(ttft, 0.9), "ttft_p99_s": pct(ttft, 0.99),
           "itl_p50_ms": 1e3 * pct(itl, 0.5) if itl else None, "itl_p90_ms": 1e3 * pct(itl, 0.9) if itl else None,
           "wall_s": total_s, "prompt_tokens": sum(lens), "layers": args.layers, "dtype": "bf16",
           "data": "synthetic prompts, random-init weights", "gpu_launches": L.LAUNCHES}
    if rank == 0:
        print(json.dumps(out))
        if args.out:
            with open(args.out, "a") as f:
                f.write(json.dumps(out) + "\n")
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    import sys
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
