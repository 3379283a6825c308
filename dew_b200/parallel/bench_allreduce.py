"""Latency of the fused all-reduce + residual add + RMSNorm kernels against NCCL all-reduce followed by the add + norm kernel.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \\
        -m dew_b200.parallel.bench_allreduce [--rows 128,2048] [--features 4096]

Each form is captured into a CUDA graph of ``--chain`` dependent calls (each call's residual is the previous call's sum, as in
a decoder), replayed ``--iters`` times, device-timed with events, and reported as microseconds per call (max over ranks).
The roofline of a call is the slower of the launch floor and the bytes one rank must send: 2 (W - 1) / W of the tensor for
a two-shot form, (W - 1) whole tensors for the one-shot pull, at the measured peer bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

PEER_GBS = 770.0            # measured peer copy bandwidth per direction on this class of machine


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", default="128,2048")
    ap.add_argument("--features", type=int, default=4096)
    ap.add_argument("--chain", type=int, default=32)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    from .. import ops
    from ..ops import library as L
    from .tp import TensorParallel

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    d = args.features
    row_counts = [int(r) for r in args.rows.split(",")]
    w = torch.ones(d, device=dev, dtype=torch.bfloat16)
    results = []

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            g.replay()
        e.record()
        torch.cuda.synchronize()
        L.check_status()
        t = torch.tensor([s.elapsed_time(e) * 1e3 / (args.iters * args.chain)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for rows in row_counts:
        part = (torch.randn(rows, d, device=dev) * 0.01).to(torch.bfloat16)
        h0 = torch.zeros(rows, d, device=dev, dtype=torch.bfloat16)
        row = {"rows": rows, "features": d, "world": world, "tensor_bytes": rows * d * 2}
        for mode in ("auto", "twoshot", "oneshot"):
            os.environ["DEWB_TP_ALLREDUCE"] = mode
            tp = TensorParallel(None, max_rows=max(row_counts), features=d, device=dev)

            def chain(tp=tp):
                h = h0
                for _ in range(args.chain):
                    n, h = tp.reduce_add_norm(part, h, w, 1e-5)
                return n
            name = {"auto": "low_latency" if rows <= tp.LL_ROWS else "two_shot", "twoshot": "two_shot", "oneshot": "one_shot"}[mode]
            if mode == "auto" and rows > tp.LL_ROWS:
                continue                                   # the same kernel as 'twoshot'
            row[name + "_us"] = timed(chain)
            del tp
        os.environ.pop("DEWB_TP_ALLREDUCE", None)

        def nccl_chain():
            h = h0
            for _ in range(args.chain):
                s = part.clone()
                dist.all_reduce(s)
                n, h = ops.stream_rms_norm(h, s, w, 1e-5)
            return n
        row["nccl_allreduce_plus_add_norm_us"] = timed(nccl_chain)
        two_shot_bytes = 2 * (world - 1) / world * rows * d * 2
        row["two_shot_link_floor_us"] = two_shot_bytes / PEER_GBS / 1e3
        row["one_shot_link_floor_us"] = (world - 1) * rows * d * 2 / PEER_GBS / 1e3
        results.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
