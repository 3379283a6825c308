"""Worker for the sharded-checkpoint test: trains a tiny LM under the FSDP engine through ``Trainer.fit`` with a
checkpoint directory, for ``steps`` steps in total (resuming whatever the directory holds), and prints the loss of every
step it ran plus a digest of the final weights (rank 0)."""
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
    directory, steps = sys.argv[1], int(sys.argv[2])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=264, emb_features=64, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=32,
                              mlp_features=128, max_seq_len=64, qk_norm=False, tie_embeddings=False)
    gen = torch.Generator().manual_seed(11)
    data = torch.randint(0, 264, (steps, 8, 65), generator=gen)       # step s always sees global batch s
    per = 8 // world

    class Stream:
        """Global batch ``position`` sliced to this rank's rows; restorable."""
        def __init__(self):
            self.i = 0
        def __iter__(self):
            return self
        def __next__(self):
            if self.i >= steps:
                raise StopIteration
            b = data[self.i, rank * per:(rank + 1) * per]
            self.i += 1
            return {"tokens": b}
        def position(self):
            return {"i": self.i}
        def restore(self, pos):
            self.i = int(pos["i"])

    ck = dew.Checkpoints(directory, keep=dew.Keep(3))
    trainer = dew.Trainer(LMObjective(model, 64, ema_decay=0.9), dew.OptimConfig(learning_rate=2e-3, weight_decay=0.01),
                          key=3, checkpoints=ck, tracker=dew.MemoryTracker())
    trainer.device = torch.device("cpu")
    trainer._engine = FSDPEngine(trainer, wait_limit_s=5.0)
    state = trainer.fit(Stream(), steps=steps, log_every=1, checkpoint_every=None, checkpoint_final=True)
    full = trainer._engine.gather_full("master")
    ema = trainer._engine.gather_full("ema")
    digest = float(sum(v.double().abs().sum() for v in full.values()))
    edigest = float(sum(v.double().abs().sum() for v in ema.values()))
    if rank == 0:
        rows = [r for r in trainer.tracker.rows if "loss" in r]
        print("RESULT " + json.dumps({"step": state.step, "digest": digest, "ema": edigest, "losses": [r["loss"] for r in rows], "world": world}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
