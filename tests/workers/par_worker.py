"""Worker for sequence-parallel attention, GPipe and DiLoCo on CPU ranks."""
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from dew_b200 import ops  # noqa: E402
from dew_b200.parallel import sp  # noqa: E402
from dew_b200.parallel.diloco import DiLoCo, DiLoCoConfig  # noqa: E402
from dew_b200.parallel.pp import GPipe, stage_slices  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, N = dist.get_rank(), dist.get_world_size()
    res = {}
    # ---- sequence-parallel attention (both schemes) against the full computation
    g = torch.Generator().manual_seed(0)
    B, S, H, Hkv, D = 2, 8 * N, 4, 2, 8
    q, k, v = (torch.randn(B, S, h, D, generator=g) for h in (H, Hkv, Hkv))
    full_in = [t.clone().requires_grad_() for t in (q, k, v)]
    ref = ops.attention_reference(*full_in, causal=True)
    ref.pow(2).sum().backward()
    loc = [t[:, rank * S // N:(rank + 1) * S // N].clone().requires_grad_() for t in (q, k, v)]
    out = sp.exchanged_heads_attention(*loc, causal=True)
    out.pow(2).sum().backward()
    sl = slice(rank * S // N, (rank + 1) * S // N)
    res["ulysses_out"] = float((out - ref[:, sl]).abs().max())
    res["ulysses_dq"] = float((loc[0].grad - full_in[0].grad[:, sl]).abs().max())
    res["ulysses_dk"] = float((loc[1].grad - full_in[1].grad[:, sl]).abs().max())
    # gathered keys with striped queries
    qs, ks, vs = (sp.stripe(t, N) for t in (q, k, v))
    pos = sp.stripe(torch.arange(S)[None, :, None].expand(B, S, 1).float(), N)[..., 0].long()
    loc2 = [t[:, sl].clone().requires_grad_() for t in (qs, ks, vs)]
    out2 = sp.gathered_keys_attention(*loc2, pos[:, sl], causal=True)
    whole = [torch.empty_like(out2) for _ in range(N)]
    dist.all_gather(whole, out2.detach())
    res["gathered_out"] = float((sp.unstripe(torch.cat(whole, 1), N) - ref.detach()).abs().max())
    # ---- GPipe over N stages equals the unsplit model
    torch.manual_seed(1)
    layers = nn.ModuleList([nn.Sequential(nn.Linear(6, 6), nn.Tanh()) for _ in range(2 * N)])
    xs = [torch.randn(3, 6, generator=torch.Generator().manual_seed(20 + i)) for i in range(4)]
    total_ref = sum(nn.Sequential(*layers)(x).pow(2).sum() for x in xs)
    ref_grads = torch.autograd.grad(total_ref, [p for l in layers for p in l.parameters()])
    mine = stage_slices(2 * N, N)[rank]
    stage = nn.Sequential(*[layers[i] for i in mine])
    for p in stage.parameters():
        p.grad = None
    loss = GPipe(stage).run(xs, lambda y, i: y.pow(2).sum(), 4, torch.empty(3, 6))
    flat_ref = [g_ for g_, (li, _) in zip(ref_grads, [(i, n) for i in range(2 * N) for n in range(2)]) if li in mine]
    res["pp_grad"] = max(float((p.grad - r).abs().max()) for p, r in zip(stage.parameters(), flat_ref))
    if rank == N - 1:
        res["pp_loss"] = abs(float(loss) - float(total_ref))
    # ---- DiLoCo: after an outer step all replicas hold the same weights
    w = nn.Parameter(torch.full((4,), 1.0))          # replicas start from the same weights
    d = DiLoCo([w], DiLoCoConfig(every=2, outer_lr=1.0, momentum=0.0, nesterov=False))
    with torch.no_grad():
        w.add_(rank + 1.0)
    d.after_inner_step()
    with torch.no_grad():
        w.add_(1.0)
    took = d.after_inner_step()
    ws = [torch.empty_like(w.data) for _ in range(N)]
    dist.all_gather(ws, w.data)
    res["diloco_spread"] = float(torch.stack(ws).std(0).max()) if N > 1 else 0.0
    res["diloco_took"] = float(took)
    gathered = [None] * N
    dist.all_gather_object(gathered, res)
    if rank == 0:
        merged = {}
        for g_ in gathered:
            for k_, v_ in g_.items():
                merged[k_] = max(merged.get(k_, 0.0), v_)
        print("RESULT " + json.dumps(merged))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
