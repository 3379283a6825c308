"""Worker: a tensor-parallel copy of a small LM must produce the same logits and greedy tokens as the unsharded one."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from dew_b200.models import CausalTransformer  # noqa: E402
from dew_b200.parallel.tp import TensorParallel, tensor_parallelize  # noqa: E402
from dew_b200.sampling.text import Sampling, generate  # noqa: E402


def main():
    backend = sys.argv[1] if len(sys.argv) > 1 else "gloo"
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
    torch.manual_seed(0)
    kw = dict(vocab_size=128, emb_features=256, num_layers=2, num_heads=8, num_kv_heads=max(4, int(os.environ.get('WORLD_SIZE', '1'))), head_dim=64, mlp_features=512,
              max_seq_len=64, qk_norm=False, tie_embeddings=False)
    full = CausalTransformer(**kw).to(dev, dtype).eval()
    torch.manual_seed(0)
    sharded = CausalTransformer(**kw).to(dev, dtype).eval()
    tp = TensorParallel(None, max_rows=256, features=256, device=dev, wait_limit_s=5.0)
    tensor_parallelize(sharded, tp)
    tokens = torch.randint(0, 128, (3, 20), generator=torch.Generator().manual_seed(5)).to(dev)
    with torch.no_grad():
        a = full(tokens).float()
        b = sharded(tokens).float()
    err = float((a - b).norm() / a.norm())
    prompts = [[5, 6, 7], [9, 10, 11, 12, 13]]
    ga = generate(full, None, prompts, 6, sampling=Sampling(temperature=0.0))
    gb = generate(sharded, None, prompts, 6, sampling=Sampling(temperature=0.0))
    same = bool(torch.equal(ga.tokens, gb.tokens))
    # the fused all-reduce + add + norm by itself: row counts that do not divide by the world, with and without residual / norm,
    # called back to back (regions rotate), against the sum computed by the process group
    worst = 0.0
    if dev.type == "cuda":
        world = dist.get_world_size()
        g = torch.Generator(device="cpu").manual_seed(100 + rank)
        w = (1.0 + 0.1 * torch.randn(256, generator=torch.Generator().manual_seed(3))).to(dev, torch.bfloat16)
        prev = None
        for it, rows in enumerate((1, 7, 60, 256, 3, 600, 128, 128, 128)):
            part = torch.randn(rows, 256, generator=g).to(dev, torch.bfloat16)
            res = None if it % 3 == 0 else torch.randn(rows, 256, generator=torch.Generator().manual_seed(50 + it)).to(dev, torch.bfloat16)
            if it >= 7:
                res = prev                                   # the residual is the previous call's own output, as in a decoder
            n, h = tp.reduce_add_norm(part, res, w if it % 2 == 0 else None, 1e-5)
            total = part.float().clone()
            dist.all_reduce(total)
            want_h = (total + (res.float() if res is not None else 0)).to(torch.bfloat16)
            worst = max(worst, float((h.float() - want_h.float()).abs().max()) / (float(want_h.float().abs().max()) + 1e-6))
            if n is not None:
                hf = want_h.float()
                want_n = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
                worst = max(worst, float((n.float() - want_n).abs().max()) / (float(want_n.abs().max()) + 1e-6))
            prev = h
    if dev.type == "cuda":
        from dew_b200.ops import library as L
        torch.cuda.synchronize()
        L.check_status()
    if rank == 0:
        print("RESULT " + json.dumps({"err": err, "same_tokens": same, "world": dist.get_world_size(), "allreduce_worst": worst}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
