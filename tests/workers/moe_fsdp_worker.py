"""Worker: a small MoE LM trained under the FSDP engine with its experts split over the ranks (expert parallelism: the
experts form rank-local units, everything else is sharded) must take the same steps as one process on the same global
batch, and its checkpoint export must hold every rank's experts."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import dew_b200 as dew  # noqa: E402
from dew_b200.models import CausalTransformer  # noqa: E402
from dew_b200.models.causal_transformer import Mixture  # noqa: E402
from dew_b200.nn.layers import reset_all  # noqa: E402
from dew_b200.objectives.lm import LMObjective  # noqa: E402
from dew_b200.parallel.ep import ExpertParallel  # noqa: E402
from dew_b200.parallel.fsdp import FSDPEngine  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    model = CausalTransformer(vocab_size=128, emb_features=64, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=32,
                              mlp_features=128, max_seq_len=32, qk_norm=False, tie_embeddings=False,
                              mixture=Mixture(experts=4, top_k=2, expert_features=32, shared_features=32))
    reset_all(model, 1234)                                   # the same full model on every rank, then split the experts
    if world > 1:
        ExpertParallel().shard(model)
    gen = torch.Generator().manual_seed(7)
    fixed = torch.randint(0, 128, (8, 33), generator=gen)
    per = 8 // world
    trainer = dew.Trainer(LMObjective(model, 32, balance=None), dew.OptimConfig(learning_rate=3e-3, weight_decay=0.01), key=3, microbatches=2)
    trainer.device = torch.device("cpu")
    engine = FSDPEngine(trainer, wait_limit_s=5.0)
    trainer._engine = engine
    if world == 1:
        # one process: keep the initial weights that reset_all(1234) drew (fresh_state would redraw from the trainer key)
        for p in model.parameters():
            p.expert_parallel = getattr(p, "expert_parallel", False)
        model.layers[0].mlp.experts.gate_up.expert_parallel = True     # marks the model as initialised already
    state = engine.fresh_state(trainer.key)
    losses = []
    for _ in range(5):
        mine = fixed[rank * per:(rank + 1) * per]
        state, metrics = engine.step(state, {"tokens": mine})
        stat = metrics["loss"]
        parts = torch.stack([stat.total.float(), stat.mass.float()])
        dist.all_reduce(parts)
        losses.append(float(parts[0] / parts[1]))
    full = engine.gather_full("master")
    digest = float(sum(v.double().abs().sum() for v in full.values()))
    experts = [tuple(v.shape) for k, v in full.items() if "gate_up" in k and "experts" in k]
    local_units = sum(u.local for u in engine.units) if world > 1 else 0
    if rank == 0:
        print("RESULT " + json.dumps({"losses": losses, "digest": digest, "experts": experts, "local_units": local_units}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
