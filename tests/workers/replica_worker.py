"""Worker: hybrid sharding (fsdp 2 x 2 replicas) trains, every rank writes a local checkpoint, one rank loses its file, and the
step is recovered from the replica that holds the same shards; then an unrecoverable loss is refused."""
import json
import os
import shutil
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import dew_b200 as dew  # noqa: E402
from dew_b200.checkpoints.replicas import ShardGrid, local_steps, restore_local, save_local  # noqa: E402
from dew_b200.models import CausalTransformer  # noqa: E402
from dew_b200.objectives.lm import LMObjective  # noqa: E402
from dew_b200.parallel.mesh import MeshSpec  # noqa: E402


def main():
    directory = sys.argv[1]
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=96, emb_features=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8,
                              mlp_features=64, max_seq_len=16, qk_norm=False, tie_embeddings=False)
    trainer = dew.Trainer(LMObjective(model, 16, ema_decay=0.9), dew.OptimConfig(learning_rate=2e-3), key=3,
                          mesh=MeshSpec(fsdp=2, replicas=2))
    engine = trainer.engine()
    state = engine.fresh_state(trainer.key)
    fixed = torch.randint(0, 96, (16, 17), generator=torch.Generator().manual_seed(7))
    per = 16 // engine.batch_ranks
    mine = {"tokens": fixed[engine.batch_index * per:(engine.batch_index + 1) * per]}
    for _ in range(2):
        state, _ = engine.step(state, mine)
    save_local(engine, state, state.step, directory)
    want = {k: t.clone() for k, t in (("master", engine.master), ("m", engine.m), ("ema", engine.ema))}
    state, _ = engine.step(state, mine)                  # the run goes on past the local step ...
    dist.barrier()
    if rank == 1:
        shutil.rmtree(os.path.join(directory, "1"))      # ... and rank 1 loses its local directory
    dist.barrier()
    grid = ShardGrid.of(engine.mesh, ("data",))
    state = restore_local(engine, state, 2, directory, grid)
    same = all(torch.equal(want[k], t) for k, t in (("master", engine.master), ("m", engine.m), ("ema", engine.ema)))
    ok = torch.tensor([1.0 if (same and state.step == 2 and int(state.opt_state["count"]) == 2) else 0.0])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    # both holders of a shard gone: refused, naming the ranks
    dist.barrier()
    holders = grid.holders[1]
    if rank in holders:
        shutil.rmtree(os.path.join(directory, str(rank)), ignore_errors=True)
    dist.barrier()
    refused = False
    try:
        restore_local(engine, state, 2, directory, grid)
    except FileNotFoundError as e:
        refused = "survive on no replica" in str(e)
    if rank == 0:
        print("RESULT " + json.dumps({"recovered": bool(ok.item() > 0), "refused": refused, "holders_of_1": list(holders),
                                      "steps_rank0": local_steps(directory, 0)}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
