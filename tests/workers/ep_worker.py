"""Worker: an expert-parallel MoE layer must reproduce the single-process layer (outputs and gradients)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from dew_b200.models.causal_transformer import Mixture  # noqa: E402
from dew_b200.nn.moe import SparseMLP  # noqa: E402
from dew_b200.parallel.ep import ExpertParallel  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    dispatch = sys.argv[1] if len(sys.argv) > 1 else "auto"
    mix = Mixture(experts=8, top_k=2, expert_features=16, shared_features=16, dispatch=dispatch)
    torch.manual_seed(0)
    full = SparseMLP(32, mix, 64)
    torch.manual_seed(0)
    sharded = SparseMLP(32, mix, 64)
    ExpertParallel().shard(sharded)
    # every rank has its own tokens
    x = torch.randn(24, 32, generator=torch.Generator().manual_seed(10 + rank), requires_grad=True)
    xs = x.detach().clone().requires_grad_()
    y_full = full(x)
    y_ep = sharded(xs)
    y_full.pow(2).sum().backward()
    y_ep.pow(2).sum().backward()
    per = 8 // world
    g_full = full.experts.gate_up.grad.clone()
    dist.all_reduce(g_full)                        # the full layer's expert gradient summed over ranks' tokens
    g_ep = sharded.experts.gate_up.grad
    res = {"out_err": float((y_full - y_ep).abs().max()), "dx_err": float((x.grad - xs.grad).abs().max()),
           "dw_err": float((g_full[rank * per:(rank + 1) * per] - g_ep).abs().max())}
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        print("RESULT " + json.dumps({k: max(g[k] for g in gathered) for k in res}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
