"""Worker for the mesh-composition tests: ``Trainer(mesh=MeshSpec(...))`` builds its own process groups and engine; a tiny LM
(or MoE LM) trains for a few steps on a fixed global batch of which every rank takes the rows of its batch coordinate.
Prints the pooled losses as JSON (rank 0)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import dew_b200 as dew  # noqa: E402
from dew_b200.models import CausalTransformer  # noqa: E402
from dew_b200.models.causal_transformer import Mixture  # noqa: E402
from dew_b200.objectives.lm import LMObjective  # noqa: E402
from dew_b200.parallel.mesh import MeshSpec  # noqa: E402


def main():
    spec = json.loads(sys.argv[1])
    optimizer = sys.argv[2] if len(sys.argv) > 2 else "adamw"
    moe = len(sys.argv) > 3 and sys.argv[3] == "moe"
    clip = float(sys.argv[4]) if len(sys.argv) > 4 and sys.argv[4] != "none" else None
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    torch.manual_seed(0)
    mix = Mixture(experts=4, top_k=2, expert_features=32, shared_features=32) if moe else None
    model = CausalTransformer(vocab_size=96, emb_features=32, num_layers=4, num_heads=4, num_kv_heads=2, head_dim=8,
                              mlp_features=64, max_seq_len=16, qk_norm=False, tie_embeddings=False, mixture=mix)
    trainer = dew.Trainer(LMObjective(model, 16, ema_decay=None),
                          dew.OptimConfig(optimizer=optimizer, learning_rate=2e-3, weight_decay=0.01, clip_grads=clip),
                          key=3, mesh=MeshSpec(**spec) if spec else None, microbatches=2)
    engine = trainer.engine()
    state = engine.fresh_state(trainer.key)
    g = torch.Generator().manual_seed(7)
    fixed = torch.randint(0, 96, (16, 17), generator=g)
    ranks, index = getattr(engine, "batch_ranks", 1), getattr(engine, "batch_index", 0)
    per = 16 // ranks
    losses = []
    for _ in range(5):
        state, metrics = engine.step(state, {"tokens": fixed[index * per:(index + 1) * per]})
        stat = metrics["loss"]
        losses.append(float(stat.total.float() / stat.mass.float()))
    # pooled over the ranks that saw different rows: the engines return their local (or already pooled) ratio; average here
    t = torch.tensor(losses, dtype=torch.float64)
    dist.all_reduce(t)
    losses = (t / dist.get_world_size()).tolist()
    if rank == 0:
        print("RESULT " + json.dumps({"losses": losses, "engine": type(engine).__name__, "step": state.step}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
