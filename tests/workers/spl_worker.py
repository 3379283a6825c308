"""Worker: the fused all-gather->GEMM and GEMM->reduce-scatter products against the unsharded fp32 products, three calls in
a row (buffer reuse), plus device timings of the fused kernels against all_gather + matmul / matmul + reduce_scatter."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from dew_b200 import ops  # noqa: E402
from dew_b200.parallel.tp import SequenceParallelLinear  # noqa: E402


def main():
    backend = sys.argv[1] if len(sys.argv) > 1 else "gloo"
    rows, K, N = (int(v) for v in (sys.argv[2:5] if len(sys.argv) > 4 else (512, 256, 384)))
    rank = int(os.environ["RANK"])
    if backend == "nccl":
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", device_id=dev)
        dtype = torch.bfloat16
    else:
        dev, dtype = torch.device("cpu"), torch.float32
        dist.init_process_group("gloo")
    W = dist.get_world_size()
    spl = SequenceParallelLinear(None, rows, K, N, device=dev, wait_limit_s=5.0)
    errs = []
    for call in range(3):
        g = torch.Generator().manual_seed(100 + call)
        x = torch.randn(rows, K, generator=g).to(dev, dtype)                    # the whole activation, same on every rank
        w_col = (torch.randn(N, K, generator=g) / K ** 0.5).to(dev, dtype)      # column-parallel weight (this rank's rows: all, for the test)
        xs = x[rank * (rows // W):(rank + 1) * (rows // W)].contiguous()
        y = spl.gather_matmul(xs, w_col)
        ref = x.float() @ w_col.float().t()
        errs.append(float((y.float() - ref).norm() / ref.norm()))
        # row-parallel: every rank holds a K-slice of x2 and of w_row; the sum over ranks is the full product
        x2 = torch.randn(rows, N, generator=g).to(dev, dtype)
        w_row = (torch.randn(K, N, generator=g) / N ** 0.5).to(dev, dtype)
        ks = N // W
        res = torch.randn(rows, K, generator=g).to(dev, dtype)
        spl2 = getattr(main, "spl2", None)
        if spl2 is None:
            spl2 = main.spl2 = SequenceParallelLinear(None, rows, ks, K, device=dev, wait_limit_s=5.0)
        mine = spl2.matmul_scatter(x2[:, rank * ks:(rank + 1) * ks].contiguous(), w_row[:, rank * ks:(rank + 1) * ks].contiguous(),
                                   res[rank * (rows // W):(rank + 1) * (rows // W)].contiguous())
        ref2 = (x2.float() @ w_row.float().t() + res.float())[rank * (rows // W):(rank + 1) * (rows // W)]
        errs.append(float((mine.float() - ref2).norm() / ref2.norm()))
    timings = {}
    if dev.type == "cuda":
        from dew_b200.ops import library as L
        torch.cuda.synchronize()
        L.check_status()
        if len(sys.argv) > 5 and sys.argv[5] == "time":
            def timed(fn, iters=10):
                for _ in range(3):
                    fn()
                dist.barrier(); torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(iters):
                    fn()
                b.record(); torch.cuda.synchronize()
                t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return float(t)
            parts = [torch.empty_like(xs) for _ in range(W)]
            def lib_ag():
                dist.all_gather(parts, xs)
                return ops.linear(torch.cat(parts, 0), w_col)
            x2s, w2s = x2[:, rank * ks:(rank + 1) * ks].contiguous(), w_row[:, rank * ks:(rank + 1) * ks].contiguous()
            out_rs = torch.empty(rows // W, K, device=dev, dtype=dtype)
            def lib_rs():
                yy = ops.linear(x2s, w2s)
                dist.reduce_scatter_tensor(out_rs, yy)
                return out_rs
            timings = {"fused_ag_gemm_ms": timed(lambda: spl.gather_matmul(xs, w_col)), "nccl_ag_then_gemm_ms": timed(lib_ag),
                       "fused_gemm_rs_ms": timed(lambda: spl2.matmul_scatter(x2s, w2s)), "gemm_then_nccl_rs_ms": timed(lib_rs)}
            torch.cuda.synchronize()
            L.check_status()
    if rank == 0:
        print("RESULT " + json.dumps({"errs": errs, "world": W, "rows": rows, "K": K, "N": N, **timings}))
    dist.barrier()
    if dev.type == "cuda":
        sys.stdout.flush()
        os._exit(0)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
