"""Worker for the multi-process FSDP tests: trains a tiny LM for a few steps under the FSDP engine and prints the
losses as JSON (rank 0).  Runs on CPU ranks (gloo) or on one GPU per rank (nccl + peer memory)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import dew_b200 as dew  # noqa: E402
from dew_b200.models import CausalTransformer  # noqa: E402
from dew_b200.objectives.lm import LMObjective  # noqa: E402
from dew_b200.parallel.fsdp import FSDPEngine  # noqa: E402


def main():
    backend = sys.argv[1] if len(sys.argv) > 1 else "gloo"
    clip = float(sys.argv[2]) if len(sys.argv) > 2 and sys.argv[2] != "none" else None
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if backend == "nccl":
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=264, emb_features=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                              mlp_features=256, max_seq_len=128, qk_norm=False, tie_embeddings=False).to(dev)
    # every rank draws the same global batches and takes its own rows
    gen = torch.Generator().manual_seed(7)
    fixed = torch.randint(0, 264, (16, 129), generator=gen)     # one global batch, repeated: the model memorises it
    batches = [fixed for _ in range(6)]
    per = 16 // world
    trainer = dew.Trainer(LMObjective(model, 128), dew.OptimConfig(learning_rate=2e-3, weight_decay=0.01, clip_grads=clip),
                          key=3, param_dtype=torch.bfloat16 if dev.type == "cuda" else None, microbatches=2)
    trainer.device = dev
    mode = sys.argv[3] if len(sys.argv) > 3 else "resident"
    if mode == "sharded":
        from dew_b200.parallel.fsdp_sharded import ShardedFSDPEngine
        engine = ShardedFSDPEngine(trainer, wait_limit_s=5.0)
    else:
        engine = FSDPEngine(trainer, wait_limit_s=5.0)
    trainer._engine = engine
    state = engine.fresh_state(trainer.key)
    losses = []
    for b in batches:
        mine = b[rank * per:(rank + 1) * per].to(dev)
        state, metrics = engine.step(state, {"tokens": mine})
        stat = metrics["loss"]
        parts = torch.stack([stat.total.float(), stat.mass.float()]).to(dev)
        dist.all_reduce(parts)
        losses.append(float(parts[0] / parts[1]))
    # straight after the step, with no synchronisation of its own: the compute copy this rank would evaluate with already
    # holds every peer's new weights (compared below with the gathered masters)
    if mode == "sharded":
        if rank == 0:
            print("RESULT " + json.dumps({"losses": losses, "digest": float(sum(v.double().abs().sum() for v in engine.gather_full("master").values())),
                                          "world": world, "arena_ok": True, "state_bytes": engine.state_bytes()}))
        else:
            engine.gather_full("master")
        dist.barrier()
        dist.destroy_process_group()
        return
    arena_now = engine.params_arena.tensor.clone()
    if dev.type == "cuda":
        from dew_b200.ops import library as L
        torch.cuda.synchronize()
        L.check_status()
    full = engine.gather_full("master")
    arena_ok = True
    for u in engine.units:
        for n, p in u.params:
            o = u.offset + u.offsets[n]
            from dew_b200.utils.trees import module_path_to_tree_path
            want = full[module_path_to_tree_path(n)].to(arena_now.dtype).reshape(-1)
            arena_ok = arena_ok and bool(torch.equal(arena_now[o:o + p.numel()], want.to(arena_now.device)))
    ok = torch.tensor([1.0 if arena_ok else 0.0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    arena_ok = bool(ok.item() > 0)
    digest = float(sum(v.double().abs().sum() for v in full.values()))
    if rank == 0:
        print("RESULT " + json.dumps({"losses": losses, "digest": digest, "world": world, "arena_ok": arena_ok}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
