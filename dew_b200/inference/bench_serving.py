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
    ap.add_argument("--out", default=None)
    ap.add_argument("--profile", default=None, help="write a torch.profiler kernel table of eight decode steps to this file")
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
    tp = TensorParallel(None, max_rows=max(args.requests, args.chunk), features=cfg["emb_features"], device=dev)
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
    start.record()
    server.run()
    end.record()
    torch.cuda.synchronize()
    L.check_status()
    ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    new_tokens = sum(len(t.tokens) for t in tickets)
    decode_tokens = server.decoded_tokens - decoded0
    ttft = sorted(t.first_token_time for t in tickets)
    out = {"metric": "TP decode tokens/sec", "value": decode_tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
           "requests": args.requests, "new_tokens_each": args.new_tokens, "decode_steps": server.steps - steps0,
           "ms_per_decode_step": ms / max(1, server.steps - steps0), "prefill_s": t_prefill,
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


if __name__ == "__main__":
    main()
