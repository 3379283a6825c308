"""The library arm of the benchmarks: the same models, batch and optimizer written with stock PyTorch only.

Nothing here imports this framework: ``nn.Linear`` (cuBLAS), ``F.scaled_dot_product_attention`` (cuDNN / flash),
``F.rms_norm``, ``F.cross_entropy``, fused ``torch.optim.AdamW``, FSDP2 (``fully_shard`` with
``MixedPrecisionPolicy(param_dtype=bf16, reduce_dtype=fp32)``) over NCCL, and for the MoE model ``torch._grouped_mm`` with
``all_to_all_single``.  It is what a PyTorch user would write for the same job (the recipe of the reference's own torch
arm: tools/reference_runs/torch_lm.py:1-40, ``--parallel fsdp2 --precision fsdp-bf16``), and it is the baseline the
framework's fused kernels are measured against on the same GPUs.

    python baseline/torch_arm.py --config dense --gpus 1 --steps 4 --warmup 3
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 baseline/torch_arm.py --config dense --gpus 8

Prints one JSON line with the fields of ``bench.py`` and ``"impl": "torch_nccl"``.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def rope_tables(seq: int, dim: int, theta: float, device):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    ang = torch.arange(seq, device=device, dtype=torch.float32)[:, None] * inv[None]
    return ang.cos(), ang.sin()


def apply_rope(x, cos, sin):
    # x [B, S, H, D]; rotate halves
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, d, hq, hkv, hd):
        super().__init__()
        self.hq, self.hkv, self.hd = hq, hkv, hd
        self.qkv = nn.Linear(d, (hq + 2 * hkv) * hd, bias=False)
        self.o = nn.Linear(hq * hd, d, bias=False)

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        qkv = self.qkv(x).view(B, S, self.hq + 2 * self.hkv, self.hd)
        q, k, v = qkv.split([self.hq, self.hkv, self.hkv], 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                           enable_gqa=self.hq != self.hkv)
        return self.o(o.transpose(1, 2).reshape(B, S, self.hq * self.hd))


class SwiGLU(nn.Module):
    def __init__(self, d, f):
        super().__init__()
        self.gate_up = nn.Linear(d, 2 * f, bias=False)
        self.down = nn.Linear(f, d, bias=False)

    def forward(self, x):
        g, u = self.gate_up(x).chunk(2, -1)
        return self.down(F.silu(g) * u)


class MoE(nn.Module):
    """Top-k softmax routing over ``experts`` SwiGLU experts split over the expert-parallel group, plus shared experts.
    Dispatch and combine are ``all_to_all_single``; the expert products are ``torch._grouped_mm``."""

    def __init__(self, d, experts, top_k, f, shared_f, group):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.E, self.k, self.f = experts, top_k, f
        self.local = experts // self.world
        self.router = nn.Linear(d, experts, bias=False)
        self.w_gate_up = nn.Parameter(torch.empty(self.local, d, 2 * f))
        self.w_down = nn.Parameter(torch.empty(self.local, f, d))
        nn.init.normal_(self.w_gate_up, std=0.02)
        nn.init.normal_(self.w_down, std=0.02)
        self.shared = SwiGLU(d, shared_f) if shared_f else None

    def forward(self, x):
        B, S, d = x.shape
        t = x.reshape(-1, d)
        probs = torch.softmax(self.router(t).float(), -1)
        w, ids = probs.topk(self.k, -1)
        w = (w / w.sum(-1, keepdim=True)).to(x.dtype)
        flat = ids.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=self.E)
        rows = t.repeat_interleave(self.k, 0)[order]
        if self.world > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)
            send = counts.view(self.world, self.local).sum(1).tolist()
            recv = recv_counts.view(self.world, self.local).sum(1).tolist()
            got = _AllToAll.apply(rows, send, recv, self.group)
            # received rows are ordered (source rank, local expert): regroup by expert
            rc = recv_counts.view(self.world, self.local)
            expert_of = torch.repeat_interleave(torch.arange(self.local, device=x.device).repeat(self.world), rc.reshape(-1))
            perm = torch.argsort(expert_of, stable=True)
            got = got[perm]
            per_expert = rc.sum(0)
        else:
            got, per_expert, perm, send, recv = rows, counts, None, None, None
        offs = torch.cumsum(per_expert, 0).to(torch.int32)
        h = torch._grouped_mm(got, self.w_gate_up.to(got.dtype), offs=offs)
        g, u = h.chunk(2, -1)
        y = torch._grouped_mm(F.silu(g) * u, self.w_down.to(got.dtype), offs=offs)
        if self.world > 1:
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(perm.numel(), device=perm.device)
            y = _AllToAll.apply(y[inv], recv, send, self.group)
        back = torch.empty_like(y)
        back[order] = y
        out = (back.view(-1, self.k, d) * w[..., None]).sum(1)
        if self.shared is not None:
            out = out + self.shared(t)
        return out.view(B, S, d)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = x.new_empty((sum(recv), x.shape[1]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send), g.shape[1]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv, group=ctx.group)
        return out, None, None, None


def gated_delta_rule(q, k, v, g, beta, chunk: int = 64):
    """Chunked gated delta rule in plain PyTorch (WY form): what a PyTorch user has without a Triton package."""
    B, T, H, D = q.shape
    q, k, v = (x.float().transpose(1, 2) for x in (q, k, v))
    g, beta = g.float().transpose(1, 2), beta.float().transpose(1, 2)
    q = q * D ** -0.5
    N = T // chunk
    rs = lambda x: x.reshape(B, H, N, chunk, *x.shape[3:])
    qc, kc, vc, gc, bc = rs(q), rs(k), rs(v), g.reshape(B, H, N, chunk).cumsum(-1), beta.reshape(B, H, N, chunk)
    kb, vb = kc * bc[..., None], vc * bc[..., None]
    tril = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    decay = torch.where(tril, (gc[..., :, None] - gc[..., None, :]).clamp(max=0).exp(), torch.zeros((), device=q.device))
    A = -(kb @ kc.transpose(-1, -2)) * decay
    A = A.masked_fill(~torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), -1), 0)
    eye = torch.eye(chunk, device=q.device)
    Tm = torch.linalg.solve_triangular(eye - A, eye.expand_as(A), upper=False)
    U, W = Tm @ vb, Tm @ (kb * gc.exp()[..., None])
    S = q.new_zeros(B, H, D, v.shape[-1])
    outs = []
    for n in range(N):
        qi, ki, gi = qc[:, :, n], kc[:, :, n], gc[:, :, n]
        attn = (qi @ ki.transpose(-1, -2)) * decay[:, :, n]
        vn = U[:, :, n] - W[:, :, n] @ S
        outs.append((qi * gi.exp()[..., None]) @ S + attn @ vn)
        gl = gi[..., -1]
        S = S * gl.exp()[..., None, None] + (ki * (gl[..., None] - gi).exp()[..., None]).transpose(-1, -2) @ vn
    return torch.stack(outs, 2).reshape(B, H, T, -1).transpose(1, 2)


class GatedDeltaNet(nn.Module):
    def __init__(self, d, heads, hd, conv):
        super().__init__()
        self.h, self.hd = heads, hd
        inner = heads * hd
        self.qkvz = nn.Linear(d, 4 * inner, bias=False)
        self.ba = nn.Linear(d, 2 * heads, bias=False)
        self.conv = nn.Conv1d(3 * inner, 3 * inner, conv, groups=3 * inner, padding=conv - 1, bias=False)
        self.A_log = nn.Parameter(torch.zeros(heads))
        self.dt_bias = nn.Parameter(torch.zeros(heads))
        self.norm_w = nn.Parameter(torch.ones(hd))
        self.out = nn.Linear(inner, d, bias=False)

    def forward(self, x, cos=None, sin=None):
        B, S, _ = x.shape
        inner = self.h * self.hd
        qkvz = self.qkvz(x)
        qkv, z = qkvz[..., :3 * inner], qkvz[..., 3 * inner:]
        qkv = F.silu(self.conv(qkv.transpose(1, 2))[..., :S]).transpose(1, 2)
        q, k, v = (t.reshape(B, S, self.h, self.hd) for t in qkv.chunk(3, -1))
        q, k = F.normalize(q.float(), dim=-1).to(x.dtype), F.normalize(k.float(), dim=-1).to(x.dtype)
        b, a = self.ba(x).chunk(2, -1)
        beta = b.sigmoid()
        g = -self.A_log.float().exp() * F.softplus(a.float() + self.dt_bias)
        o = gated_delta_rule(q, k, v, g, beta).to(x.dtype)
        o = F.rms_norm(o, (self.hd,), self.norm_w.to(o.dtype)) * F.silu(z.reshape(B, S, self.h, self.hd))
        return self.out(o.reshape(B, S, inner))


class Block(nn.Module):
    def __init__(self, cfg, kind, ep_group):
        super().__init__()
        d = cfg["d"]
        self.n1 = nn.RMSNorm(d, eps=1e-5)
        self.n2 = nn.RMSNorm(d, eps=1e-5)
        self.mixer = Attention(d, cfg["hq"], cfg["hkv"], cfg["hd"]) if kind == "attention" else \
            GatedDeltaNet(d, cfg["gdn_heads"], cfg["hd"], 4)
        m = cfg.get("moe")
        self.mlp = MoE(d, m["experts"], m["top_k"], m["f"], m["shared_f"], ep_group) if m else SwiGLU(d, cfg["f"])

    def forward(self, x, cos, sin):
        x = x + self.mixer(self.n1(x), cos, sin)
        return x + self.mlp(self.n2(x))


class LM(nn.Module):
    def __init__(self, cfg, ep_group=None):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg["vocab"], cfg["d"])
        kinds = cfg.get("kinds") or ["attention"]
        self.layers = nn.ModuleList([Block(cfg, kinds[i % len(kinds)], ep_group) for i in range(cfg["layers"])])
        self.norm = nn.RMSNorm(cfg["d"], eps=1e-5)
        self.head = nn.Linear(cfg["d"], cfg["vocab"], bias=False)

    def forward(self, tokens, cos, sin):
        h = self.embed(tokens)
        for layer in self.layers:
            h = layer(h, cos, sin)
        return self.head(self.norm(h))


CONFIGS = {
    "dense": dict(cfg=dict(vocab=128256, d=4096, layers=32, hq=32, hkv=8, hd=128, f=14336, theta=500000.0), seq=4096, rows=32,
                  metric="train tokens/sec (dense 8B LM, FSDP)", name="llama-style 8B: d4096 L32 H32/8kv ffn14336 vocab128256"),
    "moe": dict(cfg=dict(vocab=32768, d=2048, layers=24, hq=16, hkv=16, hd=128, f=1408, theta=10000.0,
                         moe=dict(experts=64, top_k=6, f=1408, shared_f=2816)), seq=4096, rows=16,
                metric="train tokens/sec (MoE LM, expert parallel)",
                name="MoE: d2048 L24 H16 64 experts x 1408 top-6 + 2 shared, bf16 expert GEMMs, vocab 32768"),
    "hybrid": dict(cfg=dict(vocab=32768, d=2048, layers=24, hq=16, hkv=16, hd=128, f=5632, theta=10000.0, gdn_heads=16,
                            kinds=["gdn", "gdn", "gdn", "attention"]), seq=8192, rows=8,
                   metric="train tokens/sec (hybrid GDN LM, FSDP)",
                   name="hybrid: d2048 L24 (3 gated-delta-net 16x128 conv4 : 1 attention), vocab 32768"),
}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="dense", choices=sorted(CONFIGS))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--micro", type=int, default=None)
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="debug only")
    ap.add_argument("--compile", action="store_true", help="torch.compile every decoder layer")
    args, _ = ap.parse_known_args(argv)
    rank, local, world = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1")))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev) if world > 1 or "RANK" in os.environ else None
    conf = CONFIGS[args.config]
    cfg = dict(conf["cfg"])
    if args.layers:
        cfg["layers"] = args.layers
    seq, rows = conf["seq"], args.rows or conf["rows"]
    micro = args.micro or {"dense": 1 if world == 1 else 2, "moe": 2, "hybrid": 1}[args.config]
    torch.manual_seed(1234)
    ep_group = dist.group.WORLD if (args.config == "moe" and world > 1) else None
    with torch.device("meta"):
        model = LM(cfg, ep_group)
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29791")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    experts = {p for n, p in model.named_parameters() if "w_gate_up" in n or "w_down" in n} if world > 1 else set()
    for layer in model.layers:
        fully_shard(layer, mp_policy=mp, ignored_params=experts or None)
    fully_shard(model, mp_policy=mp, ignored_params=experts or None)
    model.to_empty(device=dev)
    if experts:
        # materialising replaced the parameter objects: name the expert weights again
        experts = [p for n, p in model.named_parameters() if "w_gate_up" in n or "w_down" in n]
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, std=0.02)
            elif "norm" in n or n.endswith(".weight"):
                nn.init.ones_(p)
            else:
                nn.init.zeros_(p)
    if args.compile:
        for layer in model.layers:
            layer.compile()
    n_params = sum(p.numel() for p in model.parameters())
    # the expert weights are plain tensors (each rank owns its experts), everything else is sharded by FSDP2 (DTensors): the fused
    # optimizer kernel takes one kind per call, so each kind gets its own optimizer
    expert_ids = {id(p) for p in experts} if experts else set()
    rest = [p for p in model.parameters() if id(p) not in expert_ids]
    opts = [torch.optim.AdamW(rest, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)]
    if experts:
        opts.append(torch.optim.AdamW(list(experts), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True))
    cos, sin = rope_tables(seq, cfg["hd"], cfg["theta"], dev)
    gen = torch.Generator().manual_seed(1234 + rank)
    n_batches = args.warmup + 2 * args.steps + 2
    host = [torch.randint(0, cfg["vocab"], (rows, seq + 1), generator=gen).pin_memory() for _ in range(n_batches)]
    scored = rows * seq * world

    def step(tokens):
        total = torch.zeros((), device=dev)
        for i in range(0, rows, micro):
            mb = tokens[i:i + micro]
            logits = model(mb[:, :-1], cos, sin)
            loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), mb[:, 1:].reshape(-1), reduction="sum") / (rows * seq)
            loss.backward()
            total += loss.detach()
        if experts:
            # expert gradients are rank-local sums over every rank's tokens: scale like the data-parallel mean
            for p in experts:
                p.grad.div_(world)
        for o in opts:
            o.step()
            o.zero_grad(set_to_none=True)
        return total

    def sync():
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)

    device_batches = [h.to(dev) for h in host[: args.warmup + args.steps]]
    for i in range(args.warmup):
        step(device_batches[i])
    sync()
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from bench import ClockSampler                       # the clock sampler only (nvidia-smi reader; no framework code)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    s.record()
    for i in range(args.steps):
        loss = step(device_batches[args.warmup + i])
    e.record()
    sync()
    ms = s.elapsed_time(e)
    clocks = sampler.stop() if rank == 0 else None
    # end to end: pinned host tokens in, loss out, every step
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    s2.record()
    for i in range(args.steps):
        tokens = host[args.warmup + args.steps + i].to(dev, non_blocking=True)
        last = float(step(tokens).item())
    e2.record()
    sync()
    ms2 = s2.elapsed_time(e2)
    t = torch.tensor([ms, ms2], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms2 = float(t[0]), float(t[1])
    lt = loss.clone()
    dist.all_reduce(lt)
    if rank == 0:
        tokens_per_step = rows * seq * world
        print(json.dumps({
            "metric": conf["metric"], "value": tokens_per_step * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids from a seed; random-init weights)",
            "config": {"model": conf["name"], "params": n_params, "global_batch": rows * world, "seq_len": seq, "micro_batch": micro,
                       "parallelism": f"fsdp{world} (torch FSDP2)" + (f"+ep{world} (all_to_all_single + _grouped_mm)" if args.config == "moe" else ""),
                       "optimizer": "torch.optim.AdamW(fused=True), fp32 parameters and moments",
                       "l2": "inputs larger than L2 (weights stream every microbatch)", "compile": bool(args.compile)},
            "clocks": clocks,
            "e2e": {"value": tokens_per_step * args.steps / (ms2 / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": rows * (seq + 1) * 8 * world, "d2h_bytes_per_step": 4 * world, "ms_per_step": ms2 / args.steps},
            "gpu_launches": 0, "loss": float(lt), "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
            "impl": "torch_nccl", "note": "library arm: stock PyTorch modules, cuBLAS, cuDNN SDPA, FSDP2 / NCCL; none of this framework's kernels"}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
