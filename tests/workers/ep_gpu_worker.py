"""Worker (one rank per GPU): the expert-parallel layer on the peer-memory exchange kernels must reproduce the same layer
on the NCCL all-to-all path - outputs, input gradients and expert gradients - over several calls in a row."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from dew_b200.models.causal_transformer import Mixture  # noqa: E402
from dew_b200.nn.moe import SparseMLP  # noqa: E402
from dew_b200.ops import library as L  # noqa: E402
from dew_b200.parallel.ep import ExpertParallel  # noqa: E402


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    mix = Mixture(experts=16, top_k=4, expert_features=128, shared_features=0)
    layers = []
    for fused in (True, False):
        torch.manual_seed(0)
        m = SparseMLP(256, mix, 512).to(dev, torch.bfloat16)
        ExpertParallel(fused=fused).shard(m)
        if not fused:
            m.use_kernels = False
        layers.append(m)
    errs = []
    for call in range(3):
        x = torch.randn(500, 256, generator=torch.Generator().manual_seed(100 * call + rank)).to(dev, torch.bfloat16)
        xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
        ya, yb = layers[0](xa), layers[1](xb)
        dy = torch.randn(500, 256, generator=torch.Generator().manual_seed(7 + call)).to(dev, torch.bfloat16)
        for m in layers:
            m.zero_grad(set_to_none=True)
        ya.backward(dy)
        yb.backward(dy)
        L.check_status(dev)
        errs.append(max(rel(ya, yb), rel(xa.grad, xb.grad), rel(layers[0].experts.gate_up.grad, layers[1].experts.gate_up.grad),
                        rel(layers[0].experts.down.grad, layers[1].experts.down.grad),
                        rel(layers[0].router.weight.grad, layers[1].router.weight.grad)))
    gathered = [None] * world
    dist.all_gather_object(gathered, errs)
    if rank == 0:
        print("RESULT " + json.dumps({"errs": [max(g[i] for g in gathered) for i in range(3)]}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
