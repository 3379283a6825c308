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


def layer_gemm_shapes(tokens: int = 8192, d: int = 4096, qkv: int = 6144, ffn: int = 14336):
    """The twelve products of one decoder layer of the dense 8 B configuration on ``tokens`` tokens: forward, input gradient
    and weight gradient of the four projections, with the operand layouts and epilogues the training step uses (weight
    gradients accumulate into fp32)."""
    out = []
    for name, n_out, k_in in (("qkv", qkv, d), ("o", d, d), ("gate_up", 2 * ffn, d), ("down", d, ffn)):
        out.append((f"fwd {name}", tokens, n_out, k_in, False, False, torch.bfloat16, False))
        out.append((f"dgrad {name}", tokens, k_in, n_out, False, True, torch.bfloat16, False))
        out.append((f"wgrad {name}", n_out, k_in, tokens, True, True, torch.float32, True))
    return out


def bench_gemm(out, peaks, flush, shapes=None, iters=10, tokens: int = 8192):
    shapes = shapes or (layer_gemm_shapes(tokens) + [
        ("square 8192", 8192, 8192, 8192, False, False, torch.bfloat16, False),
        ("head", 4096, 128256, 4096, False, False, torch.bfloat16, False),
        ("ref 2560->9216 @24576", 24576, 9216, 2560, False, False, torch.bfloat16, False),
        ("ref 2560->64 @24576", 24576, 64, 2560, False, False, torch.bfloat16, False),
    ])
    for shape in shapes:
        name, M, N, K, a_mn, b_mn = shape[:6]
        odt, acc = (shape[6], shape[7]) if len(shape) > 6 else (torch.bfloat16, False)
        A = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
        B = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
        D = torch.zeros(M, N, device="cuda", dtype=odt)
        flops = 2.0 * M * N * K
        kw = dict(a_mn=a_mn, b_mn=b_mn, out=D, accumulate=acc)
        t = device_time(lambda: ops.gemm(A, B, kernel="sm100_tcgen05", **kw), iters=iters, flush=flush)
        c = device_time(lambda: ops.gemm(A, B, kernel="cublas", **kw), iters=iters, flush=flush)
        L.check_status()
        tf, ctf = flops / t.median_ms / 1e9, flops / c.median_ms / 1e9
        pair = {}
        if hasattr(L.load(), "dewb_gemm_pair_bf16") and N >= 256:
            ref = torch.zeros_like(D)
            ops.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=ref, kernel="sm100_tcgen05")
            p = device_time(lambda: ops.gemm(A, B, kernel="sm100_pair", **kw), iters=iters, flush=flush)
            L.check_status()
            chk = torch.zeros_like(D)
            ops.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=chk, kernel="sm100_pair")
            ptf = flops / p.median_ms / 1e9
            pair = dict(pair_ms=p.median_ms, pair_tflops=ptf, pair_frac_of_measured=ptf / peaks["bf16_tflops"],
                        pair_time_over_cublas=p.median_ms / c.median_ms, pair_equals_single=bool(torch.equal(chk, ref)))
            del ref, chk
        _row(out, kernel="gemm_sm100", name=name, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, out_dtype=str(odt).replace("torch.", ""),
             accumulate=acc, ms=t.median_ms, tflops=tf,
             frac_of_measured=tf / peaks["bf16_tflops"], cublas_ms=c.median_ms, cublas_tflops=ctf,
             time_over_cublas=t.median_ms / c.median_ms, peaks=peaks["source"], **pair)
        del A, B, D


def _raw_backward(kind, x, other, w, dy):
    """The backward launchers called directly (no autograd engine, so the call can be captured into a CUDA graph)."""
    import ctypes
    lib = L.load()
    rows, d = x.shape
    if kind == "swiglu":
        F2 = x.shape[1]
        Fh = F2 // 2
        dgu = torch.empty_like(x)

        def run():
            L.check(lib.dewb_swiglu_bwd(L.ptr(dy), L.ptr(x), ctypes.c_void_p(x.data_ptr() + Fh * 2), L.ptr(dgu),
                                        ctypes.c_void_p(dgu.data_ptr() + Fh * 2), ctypes.c_longlong(rows), ctypes.c_int(Fh),
                                        ctypes.c_longlong(F2), L.stream_ptr()), "swiglu_bwd")
        return run
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
    blocks = lib.dewb_rmsnorm_bwd_blocks(ctypes.c_longlong(rows))
    scratch = torch.empty(blocks, d, dtype=torch.float32, device=x.device)
    dx, dw = torch.empty_like(x), torch.empty(d, dtype=torch.float32, device=x.device)
    dz = torch.empty_like(x) if kind == "gated_rmsnorm" else None
    dres = dy if kind == "stream_rmsnorm" else None
    z = other if kind == "gated_rmsnorm" else None

    def run():
        L.check(lib.dewb_rmsnorm_bwd(L.ptr(dy), L.ptr(x), L.ptr(w), L.ptr(rstd), L.ptr(dres), L.ptr(z), L.ptr(dx), L.ptr(dz),
                                     L.ptr(scratch), L.ptr(dw), L.ptr(None), ctypes.c_int(0), ctypes.c_longlong(rows),
                                     ctypes.c_int(d), L.stream_ptr()), "rmsnorm_bwd")
    return run


def bench_rows(out, peaks, flush, iters=10):
    """Row kernels last tens of microseconds, so they are timed as CUDA-graph replays (no host launch overhead);
    bytes are the algorithmic minimum (each operand touched once)."""
    bw = peaks["hbm_gbs"]
    cases = [("rmsnorm", 12288, 2560), ("rmsnorm", 8192, 4096), ("stream_rmsnorm", 12288, 2560), ("stream_rmsnorm", 32768, 4096),
             ("gated_rmsnorm", 12288 * 32, 128), ("swiglu", 12288, 9216), ("swiglu", 8192, 14336)]
    for kind, rows, d in cases:
        e = rows * d * 2
        w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
        x = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
        other = torch.randn_like(x)
        with torch.no_grad():
            if kind == "rmsnorm":
                fwd, ref = (lambda: ops.rms_norm(x, w)), (lambda: ops.rms_norm_reference(x, w))
                fb, bb = 2 * e, 3 * e
            elif kind == "stream_rmsnorm":
                fwd, ref = (lambda: ops.stream_rms_norm(x, other, w)[0]), (lambda: ops.rms_norm_reference(x + other, w))
                fb, bb = 4 * e, 4 * e
            elif kind == "gated_rmsnorm":
                fwd = lambda: ops.gated_rms_norm(x, other, w)
                ref = lambda: ops.rms_norm_reference(x, w) * torch.nn.functional.silu(other)
                fb, bb = 3 * e, 5 * e
            else:
                x = torch.randn(rows, 2 * d, device="cuda").to(torch.bfloat16)
                fwd = lambda: ops.packed_swiglu(x)
                ref = lambda: torch.nn.functional.silu(x[:, :d]) * x[:, d:]
                fb, bb = 3 * e, 5 * e
            dy = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
            bwd = _raw_backward(kind, x, other, w, dy)
            t_f = device_time(fwd, iters=iters, flush=flush, graph=True)
            t_b = device_time(bwd, iters=iters, flush=flush, graph=True)
            t_ref = device_time(ref, iters=iters, flush=flush, graph=True)
        L.check_status()
        _row(out, kernel=kind, rows=rows, d=d, fwd_us=1000 * t_f.median_ms, bwd_us=1000 * t_b.median_ms,
             fwd_bwd_us=1000 * (t_f.median_ms + t_b.median_ms), torch_fwd_us=1000 * t_ref.median_ms,
             fwd_gbs=fb / t_f.median_ms / 1e6, fwd_frac_of_measured=fb / t_f.median_ms / 1e6 / bw,
             bwd_gbs=bb / t_b.median_ms / 1e6, bwd_frac_of_measured=bb / t_b.median_ms / 1e6 / bw, peaks=peaks["source"])


def bench_attention_variants(out, peaks, flush, iters=10):
    """The attention variants on the sm_100a kernels at one long row (1 x 12288 tokens, 32 / 8 heads of 128): plain causal,
    a 2048-key window, soft-capping, sinks, and the row packed as 6 documents of 2048 tokens (segment ids), forward and
    forward + backward; FLOPs count the visible (query, key) pairs only."""
    B, S, Hq, Hkv, D = 1, 12288, 32, 8, 128
    q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16).requires_grad_()
    k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
    v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
    seg = (torch.arange(S, device="cuda") // 2048 + 1).to(torch.int32)[None].expand(B, S).contiguous()
    sinks = torch.zeros(Hq, device="cuda")
    pairs_causal = S * (S + 1) / 2
    cases = [("causal", {}, pairs_causal), ("window 2048", dict(window=2048), 2048 * S - 2048 * 2047 / 2),
             ("softcap 30", dict(softcap=30.0), pairs_causal), ("sinks", dict(sinks=sinks), pairs_causal),
             ("6 packed documents", dict(segment_ids=seg), 6 * 2048 * 2049 / 2)]
    for name, kw, pairs in cases:
        o = ops.attention(q, k, v, causal=True, kernel="sm100_flash", **kw)
        do = torch.randn_like(o)
        t_f = device_time(lambda: ops.attention(q, k, v, causal=True, kernel="sm100_flash", **kw), iters=iters, flush=flush)
        t_fb = device_time(lambda: ops.attention(q, k, v, causal=True, kernel="sm100_flash", **kw).backward(do), iters=iters, flush=flush)
        L.check_status()
        flops = 4.0 * B * Hq * pairs * D
        _row(out, kernel="attention_variant", variant=name, B=B, S=S, Hq=Hq, Hkv=Hkv, D=D, fwd_ms=t_f.median_ms,
             fwd_bwd_ms=t_fb.median_ms, fwd_tflops=flops / t_f.median_ms / 1e9, fwd_bwd_tflops=3.5 * flops / t_fb.median_ms / 1e9)


def bench_attention(out, peaks, flush, iters=10, shapes=None, kernels=("sm100_flash", "sdpa")):
    import torch.nn.functional as F
    for B, S, Hq, Hkv, D in shapes or [(2, 4096, 32, 8, 128), (1, 16384, 32, 8, 128), (8, 4096, 32, 8, 128)]:
        q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16).requires_grad_()
        k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
        v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
        flops = 4.0 * B * Hq * S * S * D / 2
        row = dict(kernel="attention", B=B, S=S, Hq=Hq, Hkv=Hkv, D=D)
        with torch.no_grad():       # numerics of this library's forward against the library arm, on every run
            a = ops.attention(q, k, v, causal=True, kernel="sm100_flash").float()
            b = ops.attention(q, k, v, causal=True, kernel="sdpa").float()
            row["fwd_max_abs_diff_vs_sdpa"] = float((a - b).abs().max())
            del a, b
        for name in kernels:
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


def bench_gdn(out, peaks, flush, iters=10, shapes=None):
    """Gated delta rule, forward and forward + backward, on the reference's receipt shapes
    (src/dew/nn/kernels/fla_gdn.py:624-626: 1 x 4096, 32 and 48 value heads of 128) and the hybrid configuration's layer."""
    from ..ops import scan
    for B, T, H in shapes or [(1, 4096, 32), (1, 4096, 48), (2, 8192, 16)]:
        q = torch.nn.functional.normalize(torch.randn(B, T, H, 128, device="cuda"), dim=-1).to(torch.bfloat16).requires_grad_()
        k = torch.nn.functional.normalize(torch.randn(B, T, H, 128, device="cuda"), dim=-1).to(torch.bfloat16).requires_grad_()
        v = torch.randn(B, T, H, 128, device="cuda").to(torch.bfloat16).requires_grad_()
        g = (-torch.rand(B, T, H, device="cuda") * 0.3).requires_grad_()
        beta = torch.rand(B, T, H, device="cuda").requires_grad_()
        o, _ = scan.chunk_gated_delta_rule(q, k, v, g, beta)
        do = torch.randn_like(o)
        o.backward(do)
        L.check_status()
        t_f = device_time(lambda: scan.chunk_gated_delta_rule(q, k, v, g, beta), iters=iters, flush=flush)
        t_fb = device_time(lambda: scan.chunk_gated_delta_rule(q, k, v, g, beta)[0].backward(do), iters=iters, flush=flush)
        with torch.no_grad():
            from ..ops import gdn
            scale = 128 ** -0.5
            t_p = device_time(lambda: gdn.prepare_cuda(q, k, v, g, beta, scale, False), iters=iters, flush=flush)
            gc, W, U, P, _ = gdn.prepare_cuda(q, k, v, g, beta, scale, False)
            t_s = device_time(lambda: gdn.scan_fwd_cuda(q, k, gc, W, U, P, scale, None, False), iters=iters, flush=flush)
        L.check_status()
        _row(out, kernel="gdn", B=B, T=T, H=H, fwd_ms=t_f.median_ms, fwd_bwd_ms=t_fb.median_ms, prepare_ms=t_p.median_ms,
             scan_fwd_ms=t_s.median_ms)


def bench_ssd(out, peaks, flush, iters=10, shapes=None):
    """Mamba-2 SSD forward: the scan kernel against the loop-free chunked form in PyTorch."""
    from ..ops import scan
    for B, T, H, G in shapes or [(1, 4096, 64, 1), (2, 8192, 32, 1)]:
        x = torch.randn(B, T, H, 64, device="cuda").to(torch.bfloat16)
        dt = torch.nn.functional.softplus(torch.randn(B, T, H, device="cuda") - 2)
        A = -torch.rand(H, device="cuda") * 4 - 0.5
        Bm = (torch.randn(B, T, G, 128, device="cuda") / 8).to(torch.bfloat16)
        Cm = (torch.randn(B, T, G, 128, device="cuda") / 8).to(torch.bfloat16)
        with torch.no_grad():
            from ..ops import ssd as K
            t_k = device_time(lambda: scan.ssd(x, dt, A, Bm, Cm), iters=iters, flush=flush)
            prep = K.prepare(x, dt, A, Bm, Cm)
            t_s = device_time(lambda: K.scan_cuda(*prep, None), iters=iters, flush=flush)
            t_t = device_time(lambda: scan.ssd_chunked(x, dt, A, Bm, Cm), iters=max(2, iters // 3), flush=flush)
        L.check_status()
        _row(out, kernel="ssd", B=B, T=T, H=H, G=G, fwd_ms=t_k.median_ms, scan_kernel_ms=t_s.median_ms, torch_chunked_ms=t_t.median_ms)


def bench_sampling(out, peaks, flush, iters=10):
    """Token draws over a 128256-entry vocabulary, 128 rows: the kernels against the PyTorch transforms + multinomial."""
    from ..ops import sample as S
    from ..sampling.text import Sampling, transform_logits
    R, V = 128, 128256
    logits = torch.randn(R, V, device="cuda") * 3
    u = torch.rand(R, device="cuda")
    s = Sampling(temperature=0.8, top_k=50, top_p=0.95, min_p=0.02)
    hist, hl = torch.zeros(R, 1, dtype=torch.long, device="cuda"), torch.zeros(R, dtype=torch.long, device="cuda")

    def torch_path():
        x = transform_logits(logits, hist, hl, s, 0)
        return torch.multinomial(torch.softmax(x, -1), 1)

    t_a = device_time(lambda: S.argmax_rows(logits), iters=iters, flush=flush)
    t_ta = device_time(lambda: logits.argmax(-1), iters=iters, flush=flush)
    t_s = device_time(lambda: S.sample_rows(logits, u, s.temperature, s.top_k, s.top_p, s.min_p), iters=iters, flush=flush)
    t_ts = device_time(torch_path, iters=iters, flush=flush)
    bytes_ = R * V * 4
    _row(out, kernel="sampling", rows=R, vocab=V, argmax_ms=t_a.median_ms, argmax_gbs=bytes_ / t_a.median_ms / 1e6,
         argmax_frac_of_measured=bytes_ / t_a.median_ms / 1e6 / peaks["hbm_gbs"], torch_argmax_ms=t_ta.median_ms,
         sample_ms=t_s.median_ms, torch_filters_multinomial_ms=t_ts.median_ms)


def bench_moe(out, peaks, flush, iters=10):
    """Single-rank token exchange (config-3 layer shape: 16384 tokens x 2048, 64 experts, top 6): plan + dispatch + combine on
    the kernels against the PyTorch index-op chain."""
    from ..ops import grouped as G
    from ..ops.routing import route
    from ..parallel.ep import TokenExchange
    T, d, E, k = 16384, 2048, 64, 6
    x = torch.randn(T, d, device="cuda").to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda")
    w, ids, _ = route(logits, None, k, "softmax", True, 1.0)
    ex = TokenExchange(E, "self")
    plan = ex.plan(ids, d)
    rows = ex.push(x, plan)

    def torch_chain():
        layout = G.group_layout(ids.reshape(-1), E)
        xs = G.permute(x, layout, k)
        return G.combine(xs, layout, w, T)

    t_r = device_time(lambda: route(logits, None, k, "softmax", True, 1.0), iters=iters, flush=flush)
    t_tr = device_time(lambda: torch.topk(torch.softmax(logits, -1), k), iters=iters, flush=flush)
    t_p = device_time(lambda: ex.plan(ids, d), iters=iters, flush=flush)
    t_d = device_time(lambda: ex.push(x, plan), iters=iters, flush=flush)
    t_c = device_time(lambda: ex.pull(rows, plan, w), iters=iters, flush=flush)
    t_t = device_time(torch_chain, iters=iters, flush=flush)
    L.check_status()
    moved = T * k * d * 2
    _row(out, kernel="moe_exchange", tokens=T, d=d, experts=E, top_k=k, route_ms=t_r.median_ms, torch_softmax_topk_ms=t_tr.median_ms,
         plan_ms=t_p.median_ms, dispatch_ms=t_d.median_ms, combine_ms=t_c.median_ms, torch_layout_permute_combine_ms=t_t.median_ms,
         combine_gbs=(moved + T * d * 2) / t_c.median_ms / 1e6)


def bench_decode(out, peaks, flush, iters=10, rows=128, max_len=2304, heads=((32, 8), (4, 1))):
    """Paged decode attention at the serving configuration: 128 rows, page 64, context lengths uniform in [128, max_len], with
    the heads of one GPU (32 query / 8 KV) and of one of eight tensor-parallel ranks (4 / 1); the bytes are the keys and values
    each row reads once.  ``DEWB_DECODE_PERSIST=0`` times the one-CTA-per-chunk form instead of the balanced one."""
    from ..nn.kv_cache import KVCache, KVStore
    for Hq, Hkv in heads:
        store = KVStore(KVCache(page_size=64), 1, rows, max_len, Hkv, 128, torch.bfloat16, "cuda")
        store.k.normal_()
        store.v.normal_()
        g = torch.Generator().manual_seed(0)
        lengths = torch.randint(128, max_len + 1, (rows,), generator=g).to("cuda", torch.int32)
        q = torch.randn(rows, Hq, 128, device="cuda").to(torch.bfloat16)
        ref = store.decode_attention(0, q, lengths)
        t = device_time(lambda: store.decode_attention(0, q, lengths), iters=iters, flush=flush, graph=True)     # a launch of tens of microseconds: replayed from a graph
        L.check_status()
        nbytes = int(lengths.sum()) * Hkv * 128 * 2 * 2
        _row(out, kernel="paged_decode", rows=rows, heads=f"{Hq}/{Hkv}", max_len=max_len, mean_len=float(lengths.float().mean()), ms=t.median_ms,
             gbs=nbytes / t.median_ms / 1e6, frac_of_measured=nbytes / t.median_ms / 1e6 / peaks["hbm_gbs"], finite=bool(torch.isfinite(ref.float()).all()))


def bench_mx(out, peaks, flush, iters=10):
    """Block-scaled MXFP8 products at the expert shapes of the MoE configuration (tokens x 2816 x 2048 and tokens x 2048 x 1408),
    dense: quantiser time, product time, against this library's bf16 product of the same shape."""
    from .. import ops
    from ..ops import mx
    for M, N, K in ((16384, 2816, 2048), (16384, 2048, 1408), (98304, 2816, 2048)):
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        xq, xs = mx.quantize_mx(x)
        wq, ws = mx.quantize_mx(w, sf_rows=mx._pad128(N + mx.TILE_N))
        t_q = device_time(lambda: mx.quantize_mx(x), iters=iters, flush=flush)
        t_g = device_time(lambda: mx.gemm_mx(xq, xs, wq, ws), iters=iters, flush=flush)
        t_b = device_time(lambda: ops.linear(x, w), iters=iters, flush=flush)
        L.check_status()
        fl = 2.0 * M * N * K
        _row(out, kernel="gemm_mxfp8", M=M, N=N, K=K, quantize_ms=t_q.median_ms, quantize_gbs=(M * K * 3 + M * K / 32) / t_q.median_ms / 1e6,
             ms=t_g.median_ms, tflops=fl / t_g.median_ms / 1e9, bf16_ms=t_b.median_ms, bf16_tflops=fl / t_b.median_ms / 1e9,
             frac_of_measured_bf16_peak=fl / t_g.median_ms / 1e9 / peaks["bf16_tflops"])


def bench_conv(out, peaks, flush, iters=10):
    """Depthwise causal short convolution (kernel 4, SiLU) at the hybrid configuration's layer: 8 x 8192 tokens x 6144 channels."""
    from ..ops.conv import short_conv_cuda
    B, T, C, K = 8, 8192, 6144, 4
    x = torch.randn(B, T, C, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = torch.randn(C, K, device="cuda").to(torch.bfloat16).requires_grad_(True)
    t_f = device_time(lambda: short_conv_cuda(x.detach(), w.detach()), iters=iters, flush=flush)
    dy = torch.randn(B, T, C, device="cuda").to(torch.bfloat16)

    def both():
        x.grad = None
        w.grad = None
        short_conv_cuda(x, w).backward(dy)
    t_b = device_time(both, iters=iters, flush=flush)
    L.check_status()
    nbytes = B * T * C * 2
    _row(out, kernel="short_conv", B=B, T=T, C=C, K=K, fwd_ms=t_f.median_ms, fwd_gbs=2 * nbytes / t_f.median_ms / 1e6,
         fwd_frac_of_measured=2 * nbytes / t_f.median_ms / 1e6 / peaks["hbm_gbs"], fwd_bwd_ms=t_b.median_ms)


def bench_decode_gemm(out, peaks, flush, iters=10):
    """The four projections of a decode step (128 rows) of the dense 8 B decoder, per tensor-parallel degree 8 / 2 / 1: the
    weight-streaming kernel (with the SwiGLU epilogue for gate | up) against the library arm (cuBLAS through torch.matmul, plus
    this library's SwiGLU kernel where the epilogue would have done it); CUDA-graph replays, L2 flushed; the bytes are the weight."""
    from ..ops import functional as Fn
    d, F, Hq, Hkv, D = 4096, 14336, 32, 8, 128
    for tp in (8, 2, 1):
        shapes = [("qkv", (Hq + 2 * Hkv) * D // tp, d, False), ("o", d, Hq * D // tp, False), ("gate_up+swiglu", F // tp, d, True),
                  ("down", d, F // tp, False)]
        for name, N, K, glu in shapes:
            x = torch.randn(128, K, device="cuda").to(torch.bfloat16)
            w = (torch.randn((2 * N if glu else N), K, device="cuda") * 0.02).to(torch.bfloat16)
            with torch.no_grad():
                if glu:
                    mine = lambda: ops.linear_swiglu(x, w, fused=True)
                    lib = lambda: ops.packed_swiglu(torch.matmul(x, w.t()))
                else:
                    mine = lambda: ops.gemm(x, w, kernel="sm100_skinny")
                    lib = lambda: torch.matmul(x, w.t())
                t_m = device_time(mine, iters=iters, flush=flush, graph=True)
                t_l = device_time(lib, iters=iters, flush=flush, graph=True)
            L.check_status()
            nbytes = w.numel() * 2
            _row(out, kernel="decode_gemm", tp=tp, product=name, N=N, K=K, weight_mb=nbytes / 1e6, split=Fn.skinny_split(N, K, 64 if glu else 128),
                 skinny_us=t_m.median_ms * 1e3, library_us=t_l.median_ms * 1e3, skinny_gbs=nbytes / t_m.median_ms / 1e6,
                 skinny_frac_of_measured=nbytes / t_m.median_ms / 1e6 / peaks["hbm_gbs"], library_over_skinny=t_l.median_ms / t_m.median_ms)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--only", default="gemm,rows,attention")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gemm-shape", default=None, help="M,N,K[,a_mn,b_mn]: time one GEMM shape only (small profiling case)")
    ap.add_argument("--tokens", type=int, default=8192, help="gemm: tokens per microbatch of the layer shapes (8192 on one GPU, 16384 from two)")
    ap.add_argument("--decode-heads", default=None, help="Hq,Hkv: time the paged decode kernel with these head counts only (small profiling case)")
    ap.add_argument("--gdn-shape", default=None, help="B,T,H: time the gated-delta-rule kernels on one shape only (small profiling case)")
    ap.add_argument("--attn-shape", default=None, help="B,S,Hq,Hkv,D: time this library's attention kernels on one shape only")
    ap.add_argument("--flash-variant", type=int, default=None, help="forward variant: 0 = P through shared memory, 1 = P in tensor memory")
    args = ap.parse_args(argv)
    if args.flash_variant is not None:
        L.load().dewb_flash_set_variant(int(args.flash_variant))
    peaks = measured_peaks()
    flush = L2Flush()
    out = open(args.out, "a") if args.out else None
    only = args.only.split(",")
    if args.gemm_shape:
        f = [int(x) for x in args.gemm_shape.split(",")]
        f += [0] * (5 - len(f))
        bench_gemm(out, peaks, flush, shapes=[("custom", f[0], f[1], f[2], bool(f[3]), bool(f[4]))], iters=args.iters)
        return
    if args.gdn_shape:
        bench_gdn(out, peaks, flush, iters=args.iters, shapes=[tuple(int(x) for x in args.gdn_shape.split(","))])
        return
    if args.attn_shape:
        bench_attention(out, peaks, flush, iters=args.iters, shapes=[tuple(int(x) for x in args.attn_shape.split(","))],
                        kernels=("sm100_flash",))
        return
    if "gemm" in only:
        bench_gemm(out, peaks, flush, iters=args.iters, tokens=args.tokens)
    if "rows" in only:
        bench_rows(out, peaks, flush, iters=args.iters)
    if "attention" in only:
        bench_attention(out, peaks, flush, iters=args.iters)
    if "attention_variants" in only:
        bench_attention_variants(out, peaks, flush, iters=args.iters)
    if "gdn" in only:
        bench_gdn(out, peaks, flush, iters=args.iters)
    if "ssd" in only:
        bench_ssd(out, peaks, flush, iters=args.iters)
    if "sampling" in only:
        bench_sampling(out, peaks, flush, iters=args.iters)
    if "moe" in only:
        bench_moe(out, peaks, flush, iters=args.iters)
    if "decode_gemm" in only:
        bench_decode_gemm(out, peaks, flush, iters=args.iters)
    if "mx" in only:
        bench_mx(out, peaks, flush, iters=args.iters)
    if "conv" in only:
        bench_conv(out, peaks, flush, iters=args.iters)
    if "decode" in only:
        heads = ((32, 8), (4, 1)) if not args.decode_heads else (tuple(int(v) for v in args.decode_heads.split(",")),)
        bench_decode(out, peaks, flush, iters=args.iters, heads=heads)


if __name__ == "__main__":
    main()
