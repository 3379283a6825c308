"""Kernel micro-benchmarks with roofline fractions: ``python -m dew_b200.telemetry.kernel_bench [--out file.jsonl]``.

Each row: kernel, shape, median device ms, achieved TFLOP/s or GB/s, the fraction "of measured" peak, and the
library arm (cuBLAS / torch) on the same shape.  Shapes are the reference's receipt shapes
(src/dew/nn/kernels/norm_swiglu.py:560-566, grouped_matmul.py:2184-2191) and the config-2 layer shapes.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .. import ops
from ..ops import library as L
from .benchmark import L2Flush, device_time, measured_peaks


def _row(out, **kw):
    print(json.dumps(kw), flush=True)
    if out is not None:
        out.write(json.dumps(kw) + "\n")
        out.flush()


def bench_gemm(out, peaks, flush, shapes=None, iters=10):
    shapes = shapes or [
        ("fwd qkv", 8192, 6144, 4096, False, False), ("fwd o", 8192, 4096, 4096, False, False),
        ("fwd gate_up", 8192, 28672, 4096, False, False), ("fwd down", 8192, 4096, 14336, False, False),
        ("dgrad gate_up", 8192, 4096, 28672, False, True), ("wgrad gate_up", 28672, 4096, 8192, True, True),
        ("wgrad down", 4096, 14336, 8192, True, True), ("square 8192", 8192, 8192, 8192, False, False),
        ("head", 4096, 128256, 4096, False, False),
        ("ref 2560->9216 @24576", 24576, 9216, 2560, False, False), ("ref 2560->64 @24576", 24576, 64, 2560, False, False),
    ]
    for name, M, N, K, a_mn, b_mn in shapes:
        A = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
        B = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
        D = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        t = device_time(lambda: ops.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=D, kernel="sm100_tcgen05"), iters=iters, flush=flush)
        c = device_time(lambda: ops.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=D, kernel="cublas"), iters=iters, flush=flush)
        L.check_status()
        tf, ctf = flops / t.median_ms / 1e9, flops / c.median_ms / 1e9
        _row(out, kernel="gemm_sm100", name=name, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, ms=t.median_ms, tflops=tf,
             frac_of_measured=tf / peaks["bf16_tflops"], cublas_ms=c.median_ms, cublas_tflops=ctf,
             time_over_cublas=t.median_ms / c.median_ms, peaks=peaks["source"])
        del A, B, D


def bench_rows(out, peaks, flush, iters=10):
    bw = peaks["hbm_gbs"]
    cases = [("rmsnorm", 12288, 2560), ("rmsnorm", 8192, 4096), ("stream_rmsnorm", 12288, 2560), ("stream_rmsnorm", 32768, 4096),
             ("gated_rmsnorm", 12288 * 32, 128), ("swiglu", 12288, 9216), ("swiglu", 8192, 14336)]
    for kind, rows, d in cases:
        x = torch.randn(rows, d, device="cuda").to(torch.bfloat16).requires_grad_()
        w = torch.ones(d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        if kind == "rmsnorm":
            fwd = lambda: ops.rms_norm(x, w)
            ref = lambda: ops.rms_norm_reference(x, w)
            fb, bb = 2 * rows * d * 2, 3 * rows * d * 2
        elif kind == "stream_rmsnorm":
            b = torch.randn_like(x)
            fwd = lambda: ops.stream_rms_norm(x, b, w)[0]
            ref = lambda: ops.rms_norm_reference(x + b, w)
            fb, bb = 4 * rows * d * 2, 3 * rows * d * 2
        elif kind == "gated_rmsnorm":
            z = torch.randn_like(x).requires_grad_()
            fwd = lambda: ops.gated_rms_norm(x, z, w)
            ref = lambda: ops.rms_norm_reference(x, w) * torch.nn.functional.silu(z)
            fb, bb = 3 * rows * d * 2, 5 * rows * d * 2
        else:
            gu = torch.randn(rows, 2 * d, device="cuda").to(torch.bfloat16).requires_grad_()
            fwd = lambda: ops.packed_swiglu(gu)
            ref = lambda: torch.nn.functional.silu(gu[:, :d]) * gu[:, d:]
            fb, bb = 3 * rows * d * 2, 5 * rows * d * 2
        y = fwd()
        dy = torch.randn_like(y)
        def fb():
            for t in (x, w):
                t.grad = None
            fwd().backward(dy)
        # row kernels last tens of microseconds: time CUDA-graph replays so host launch overhead is excluded
        t_f = device_time(lambda: fwd(), iters=iters, flush=flush, graph=True)
        t_fb = device_time(fb, iters=iters, flush=flush, graph=True)
        t_ref = device_time(lambda: ref(), iters=iters, flush=flush, graph=True)
        L.check_status()
        _row(out, kernel=kind, rows=rows, d=d, fwd_us=1000 * t_f.median_ms, fwd_bwd_us=1000 * t_fb.median_ms,
             torch_fwd_us=1000 * t_ref.median_ms, fwd_gbs=fb / t_f.median_ms / 1e6,
             fwd_frac_of_measured=fb / t_f.median_ms / 1e6 / bw,
             bwd_gbs=bb / max(t_fb.median_ms - t_f.median_ms, 1e-6) / 1e6, peaks=peaks["source"])


def bench_attention(out, peaks, flush, iters=10):
    import torch.nn.functional as F
    for B, S, Hq, Hkv, D in [(2, 4096, 32, 8, 128), (1, 16384, 32, 8, 128), (8, 4096, 32, 8, 128)]:
        q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16).requires_grad_()
        k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
        v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
        flops = 4.0 * B * Hq * S * S * D / 2
        row = dict(kernel="attention", B=B, S=S, Hq=Hq, Hkv=Hkv, D=D)
        for name in ("sm100_flash", "sdpa"):
            try:
                o = ops.attention(q, k, v, causal=True, kernel=name)
            except Exception as e:
                row[f"{name}_error"] = str(e)[:120]
                continue
            do = torch.randn_like(o)
            try:
                L.check_status()
                ops.attention(q, k, v, causal=True, kernel=name).backward(do)
                L.check_status()            # never time a kernel that has just reported a timed-out wait
            except Exception as e:
                row[f"{name}_error"] = str(e)[:120]
                continue
            t_f = device_time(lambda: ops.attention(q, k, v, causal=True, kernel=name), iters=iters, flush=flush)
            t_fb = device_time(lambda: ops.attention(q, k, v, causal=True, kernel=name).backward(do), iters=iters, flush=flush)
            row[f"{name}_fwd_ms"], row[f"{name}_fwd_bwd_ms"] = t_f.median_ms, t_fb.median_ms
            row[f"{name}_fwd_tflops"] = flops / t_f.median_ms / 1e9
            row[f"{name}_fwd_bwd_tflops"] = 3.5 * flops / t_fb.median_ms / 1e9
        L.check_status()
        _row(out, **row)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--only", default="gemm,rows,attention")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gemm-shape", default=None, help="M,N,K[,a_mn,b_mn]: time one GEMM shape only (small profiling case)")
    args = ap.parse_args(argv)
    peaks = measured_peaks()
    flush = L2Flush()
    out = open(args.out, "a") if args.out else None
    only = args.only.split(",")
    if args.gemm_shape:
        f = [int(x) for x in args.gemm_shape.split(",")]
        f += [0] * (5 - len(f))
        bench_gemm(out, peaks, flush, shapes=[("custom", f[0], f[1], f[2], bool(f[3]), bool(f[4]))], iters=args.iters)
        return
    if "gemm" in only:
        bench_gemm(out, peaks, flush, iters=args.iters)
    if "rows" in only:
        bench_rows(out, peaks, flush, iters=args.iters)
    if "attention" in only:
        bench_attention(out, peaks, flush, iters=args.iters)


if __name__ == "__main__":
    main()
