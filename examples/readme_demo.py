"""The canonical tour: train a small LM, resume it from its checkpoint, tune it with DPO on synthetic preferences, then
train a flow-matching DiT and draw a preview grid.  Runs on CPU in well under a minute; on a B200 every hot op takes
the sm_100a kernels.  Counterpart of the reference's examples/readme_demo.py:41-138.

    python examples/readme_demo.py [--device cuda] [--out runs/demo]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))     # run from a checkout without installing

import dew_b200 as dew
from dew_b200.diffusion import Flow
from dew_b200.models import CausalTransformer, SimpleDiT
from dew_b200.objectives.diffusion import DiffusionObjective
from dew_b200.objectives.lm import LMObjective
from dew_b200.objectives.rl import DPO


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default="runs/demo")
    args = ap.parse_args()
    dev = torch.device(args.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    torch.manual_seed(0)

    # 1. language model on byte tokens
    text = ("the quick brown fox jumps over the lazy dog. " * 200).encode()
    tokens = torch.tensor(list(text), dtype=torch.long)
    windows = tokens[: (len(tokens) // 65) * 65].view(-1, 65)
    model = CausalTransformer(vocab_size=256, emb_features=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64 if dev.type == "cuda" else 32,
                              mlp_features=256, max_seq_len=64, qk_norm=False).to(dev)
    ck = dew.Checkpoints(os.path.join(args.out, "lm"), keep=dew.Keep(2))
    trainer = dew.Trainer(LMObjective(model, 64), dew.OptimConfig(learning_rate=3e-3), checkpoints=ck, tracker=dew.MemoryTracker(),
                          param_dtype=dtype if dev.type == "cuda" else None)
    data = dew.Memory({"tokens": windows}).shuffle(0).repeat().batched(16)
    state = trainer.fit(data, steps=30, log_every=10)
    print("lm loss:", [round(r["loss"], 3) for r in trainer.tracker.rows if "loss" in r])

    # 2. resume: a fresh trainer over the same directory continues at step 30
    trainer2 = dew.Trainer(LMObjective(model, 64), dew.OptimConfig(learning_rate=3e-3), checkpoints=ck, tracker=dew.MemoryTracker(),
                           param_dtype=dtype if dev.type == "cuda" else None)
    state = trainer2.fit(data, steps=40, log_every=10)
    print("resumed to step", state.step)

    # 3. DPO on synthetic preferences: "chosen" continues the pangram, "rejected" is noise
    chosen = windows[:32, :48]
    rejected = torch.cat([windows[:32, :16], torch.randint(97, 123, (32, 32))], 1)
    mask = torch.ones(32, 48, dtype=torch.long); mask[:, :16] = 0                 # score the continuation, not the prompt
    prefs = dew.Memory({"chosen": chosen, "chosen_mask": mask, "rejected": rejected, "rejected_mask": mask}).repeat().batched(8)
    dpo = dew.Trainer(DPO(model, beta=0.1), dew.OptimConfig(learning_rate=1e-4), tracker=dew.MemoryTracker(),
                      param_dtype=dtype if dev.type == "cuda" else None)
    dpo.fit(prefs, steps=10, log_every=5)
    print("dpo loss:", [round(r["loss"], 4) for r in dpo.tracker.rows if "loss" in r])

    # 4. flow-matching DiT on synthetic images, preview grid from the EMA weights
    dit = SimpleDiT(patch_size=4, emb_features=64, num_layers=2, num_heads=2 if dev.type == "cpu" else 1).to(dev)
    obj = DiffusionObjective(dit, Flow(), dew.InputSpec(dew.Field("sample", (16, 16, 3))), ema_decay=0.99)
    images = dew.Memory({"sample": torch.rand(64, 16, 16, 3) * 2 - 1}).repeat().batched(16)
    dt = dew.Trainer(obj, dew.OptimConfig(learning_rate=2e-4), tracker=dew.MemoryTracker())
    st = dt.fit(images, steps=20, log_every=10)
    grid = obj.generate(st.averaged, (4, 16, 16, 3), key=0, steps=8, solver=dew.Euler())
    print("preview grid:", tuple(grid.shape), "range", float(grid.min()), float(grid.max()))


if __name__ == "__main__":
    main()
