"""A mixture-of-experts LM over several ranks: experts split over the ranks (expert parallelism, tokens exchanged between
ranks), everything else sharded by the FSDP engine.  One process per rank:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29555 \
        examples/moe_mesh.py [--steps 30] [--backend gloo|nccl]

On GPUs (``--backend nccl``) the token exchange runs over peer memory; on CPU ranks (``gloo``) it is the all-to-all form
of the same protocol.  Counterpart of the reference's examples/moe_mesh.py.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.models import CausalTransformer
from dew_b200.models.causal_transformer import Mixture
from dew_b200.nn.layers import reset_all
from dew_b200.objectives.lm import LMObjective
from dew_b200.parallel.ep import ExpertParallel
from dew_b200.parallel.fsdp import FSDPEngine


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--backend", default="nccl" if torch.cuda.is_available() else "gloo")
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if args.backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    # the same seed on every rank: all build the same model, then each keeps its own experts
    model = CausalTransformer(vocab_size=256, emb_features=64, num_layers=2, num_heads=2, head_dim=32, mlp_features=128, max_seq_len=64,
                              qk_norm=False, tie_embeddings=False,
                              mixture=Mixture(experts=4 * world, top_k=2, expert_features=64, shared_features=64)).to(dev)
    reset_all(model, 1234)
    if world > 1:
        ExpertParallel().shard(model)
    trainer = dew.Trainer(LMObjective(model, 64, ema_decay=None, balance=0.01), dew.OptimConfig(learning_rate=3e-3), key=0,
                          param_dtype=torch.bfloat16 if dev.type == "cuda" else None)
    trainer.device = dev
    engine = FSDPEngine(trainer)
    trainer._engine = engine
    state = engine.fresh_state(trainer.key)
    text = torch.tensor(list((b"the quick brown fox jumps over the lazy dog. " * 200)), dtype=torch.long)
    windows = text[: (len(text) // 65) * 65].view(-1, 65)
    per = 8
    losses = []
    for step in range(args.steps):
        rows = windows[((step * world + rank) * per) % (len(windows) - per):][:per].to(dev)      # every rank reads its own rows
        state, metrics = engine.step(state, {"tokens": rows})
        stat = metrics["loss"]
        parts = torch.stack([stat.total.float(), stat.mass.float()]).to(dev)
        dist.all_reduce(parts)
        losses.append(float(parts[0] / parts[1]))
    if rank == 0:
        print("RESULT " + json.dumps({"world": world, "first": losses[0], "last": losses[-1]}))
    dist.barrier()
    dist.destroy_process_group()
    return losses


if __name__ == "__main__":
    main()
