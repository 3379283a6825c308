"""The run inspector reports each group's parameter norm and the update it took."""
from types import SimpleNamespace

import torch

from dew_b200.training.inspection import RunInspector, group_of


def test_groups_and_update_ratios():
    assert group_of("params.layers.3.mixer.qkv_proj.weight") == "layers.3" and group_of("embed.weight") == "embed"
    assert group_of("params.final_norm.weight") == "final_norm"
    params = {"layers": {"0": {"w": torch.ones(4, 4)}, "1": {"w": torch.full((4, 4), 2.0)}}, "embed": {"weight": torch.ones(8)}}
    state = SimpleNamespace(step=10, variables={"params": params})
    ins = RunInspector(every=10)
    ins(state)
    assert ins.summaries() == {}
    stepped = {"layers": {"0": {"w": torch.ones(4, 4) * 1.01}, "1": {"w": torch.full((4, 4), 2.0)}}, "embed": {"weight": torch.ones(8) - 0.5}}
    ins(SimpleNamespace(step=11, variables={"params": stepped}))
    s = ins.summaries()
    assert abs(s["inspect/layers.0/update_ratio"] - 0.01 / 1.01) < 1e-5 and s["inspect/layers.1/update_ratio"] == 0.0
    assert abs(s["inspect/embed/update_rms"] - 0.5) < 1e-6 and abs(s["inspect/max_update_ratio"] - 1.0) < 1e-6 and ins.worst_group == "embed"
    ins(SimpleNamespace(step=12, variables={"params": stepped}))           # not a step to look at: nothing changes
    assert len(ins.rows) == 1


def test_inspector_rides_a_fit():
    import dew_b200 as dew
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=32, emb_features=16, num_layers=2, num_heads=2, mlp_features=32, max_seq_len=16)
    trainer = dew.Trainer(LMObjective(model, 8), dew.OptimConfig(learning_rate=1e-2))
    data = dew.Memory({"tokens": torch.randint(0, 32, (64, 9))}).repeat().batched(8)
    ins = RunInspector(every=2)
    rows = []
    trainer.fit(data, steps=6, log_every=2, observe=ins, summaries=ins.summaries, log=rows.append) if "log" in trainer.fit.__code__.co_varnames else \
        trainer.fit(data, steps=6, log_every=2, observe=ins, summaries=ins.summaries)
    assert len(ins.rows) >= 2 and ins.rows[-1]["inspect/max_update_ratio"] > 0
    assert any(k.startswith("inspect/layers_0/") for k in ins.rows[-1])
