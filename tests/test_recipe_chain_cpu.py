"""The chained recipe: pre-training, SFT under a loss mask, DPO and GRPO stages over one model, each starting from the last."""
import importlib.util
import os

import torch

import dew_b200 as dew
from dew_b200.models import CausalTransformer


def _load():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "recipes", "chain.py")
    spec = importlib.util.spec_from_file_location("recipe_chain", path)
    mod = importlib.util.module_from_spec(spec)
    import sys
    sys.modules["recipe_chain"] = mod                 # dataclasses resolve their annotations through sys.modules
    spec.loader.exec_module(mod)
    return mod


def test_chain_runs_four_stages_over_one_model(tmp_path):
    chain = _load()
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    model = CausalTransformer(vocab_size=32, emb_features=48, num_layers=2, num_heads=2, head_dim=24, mlp_features=96, max_seq_len=16, qk_norm=False)

    def sums(n):
        a, b = torch.randint(0, 5, (n,), generator=g), torch.randint(0, 5, (n,), generator=g)
        return a, b
    # tokens: digits 0-9 -> ids 10-19, '+' 20, '=' 21, end 22
    def row(a, b, answer=None):
        ans = int(a + b) if answer is None else int(answer)
        return [10 + int(a), 20, 10 + int(b), 21, 10 + ans, 22]
    a, b = sums(512)
    pre = [{"tokens": torch.tensor([row(x, y) for x, y in zip(a[i:i + 64], b[i:i + 64])])} for i in range(0, 512, 64)]
    mask = torch.zeros(64, 6)
    mask[:, 4:] = 1                                                   # the answer and the end token only
    sft = [{**bt, "loss_mask": mask.clone()} for bt in pre[:4]]
    a2, b2 = sums(128)
    chosen = torch.tensor([row(x, y) for x, y in zip(a2, b2)])
    rejected = torch.tensor([row(x, y, (int(x + y) + 1) % 10) for x, y in zip(a2, b2)])
    pm = torch.zeros(128, 6)
    pm[:, 4:] = 1
    pairs = [{"chosen": chosen[i:i + 32], "rejected": rejected[i:i + 32], "chosen_mask": pm[i:i + 32], "rejected_mask": pm[i:i + 32]} for i in range(0, 128, 32)]
    prompts = [row(x, y)[:4] for x, y in zip(*sums(64))]
    reward = lambda p, c: float(len(c) >= 1 and c[0] == 10 + (p[0] - 10) + (p[2] - 10))
    recipe = chain.Recipe(model, [
        chain.Stage("pretrain", "lm", data=pre, steps=300, optimizer=dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0)),
        chain.Stage("sft", "sft", data=sft, steps=30, optimizer=dew.OptimConfig(learning_rate=1e-3, weight_decay=0.0)),
        chain.Stage("prefer", "dpo", data=pairs, steps=20, optimizer=dew.OptimConfig(learning_rate=3e-4, weight_decay=0.0), options={"beta": 0.5}),
        chain.Stage("rl", "grpo", prompts=prompts, reward=reward, steps=8, max_new_tokens=2, options={"group": 4, "kl": 0.0},
                    optimizer=dew.OptimConfig(learning_rate=1e-4, weight_decay=0.0)),
    ], directory=str(tmp_path), key=0)
    report = recipe.run()
    assert [r["stage"] for r in report] == ["pretrain", "sft", "prefer", "rl"]
    assert report[0]["loss_last"] < 0.6 * report[0]["loss_first"]
    # each stage started from the last one's weights: the SFT stage's first loss is already low, not a fresh model's
    assert report[1]["loss_first"] < 0.5 * report[0]["loss_first"]
    assert report[3]["reward_last"] > 0.6 and report[3]["steps"] == 8
    assert sorted(os.listdir(tmp_path)) == ["0-pretrain", "1-sft", "2-prefer", "3-rl"]
    import pytest
    with pytest.raises(ValueError):
        chain.Stage("x", "grpo")
    with pytest.raises(ValueError):
        chain.Stage("x", "ppo", data=[])
