"""Objectives beyond diffusion / LM: supervised, JEPA, DPO, GRPO, PPO, distillation; placement report."""
import torch
import torch.nn as nn

import dew_b200 as dew
from dew_b200.models import CausalTransformer
from dew_b200.objectives.distillation import Distillation
from dew_b200.objectives.jepa import JepaModel, JepaObjective, MultiBlockMask
from dew_b200.objectives.rl import DPO, GRPO, PPO
from dew_b200.objectives.rl.policy import gae, group_advantages
from dew_b200.objectives.supervised import Supervised
from dew_b200.parallel.layout import Layout, placement_report
from dew_b200.parallel.mesh import MeshSpec


def _lm(seed=0):
    torch.manual_seed(seed)
    return CausalTransformer(vocab_size=50, emb_features=32, num_layers=1, num_heads=4, mlp_features=64, max_seq_len=32)


def test_supervised_learns():
    torch.manual_seed(0)
    x = torch.randn(64, 8)
    y = (x[:, 0] > 0).long()
    model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 2))
    tr = dew.Trainer(Supervised(model), dew.OptimConfig(learning_rate=5e-2, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    tr.fit(dew.Memory({"inputs": x, "targets": y}).repeat().batched(32), steps=40, log_every=10)
    assert t.rows[-1]["loss"] < t.rows[0]["loss"] and t.rows[-1]["accuracy"] > 0.8


def test_jepa_target_encoder_lives_in_the_ema_slot():
    torch.manual_seed(0)
    enc = nn.Sequential(nn.Linear(12, 16), nn.GELU(), nn.Linear(16, 16))
    pred = nn.Sequential(nn.Linear(16, 16), nn.GELU(), nn.Linear(16, 16))
    obj = JepaObjective(JepaModel(enc, pred, 16), MultiBlockMask(grid=(4, 4), targets=2))
    tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=1e-2), tracker=(t := dew.MemoryTracker()))
    data = dew.Memory({"sample": torch.randn(32, 16, 12)}).repeat().batched(8)
    st = tr.fit(data, steps=10, log_every=5)
    assert st.ema is not None and "effective_rank" in t.rows[-1]
    c, tg = MultiBlockMask(grid=(6, 6)).sample(3)
    assert not bool((c & tg).any()) and bool(c.any()) and bool(tg.any())


def test_dpo_prefers_chosen():
    m = _lm()
    obj = DPO(m, beta=0.5)
    g = torch.Generator().manual_seed(1)
    chosen, rejected = torch.randint(0, 50, (8, 12), generator=g), torch.randint(0, 50, (8, 12), generator=g)
    mask = torch.ones(8, 12, dtype=torch.long); mask[:, :4] = 0
    batch = {"chosen": chosen, "chosen_mask": mask, "rejected": rejected, "rejected_mask": mask}
    tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=5e-3, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    tr.fit(dew.Loader(lambda part: iter([batch] * 30), batch=8), steps=20, log_every=5)
    assert t.rows[-1]["reward_accuracy"] >= t.rows[0]["reward_accuracy"] and t.rows[-1]["loss"] < t.rows[0]["loss"]


def test_grpo_and_ppo_losses_and_advantages():
    a = group_advantages(torch.tensor([1.0, 0.0, 0.0, 1.0, 2.0, 2.0, 2.0, 2.0]), 4)
    assert abs(float(a[:4].sum())) < 1e-5 and torch.allclose(a[4:], torch.zeros(4), atol=1e-3)
    adv, ret = gae(torch.ones(3, 2), torch.zeros(4, 2), torch.zeros(3, 2), gamma=1.0, lam=1.0)
    assert torch.allclose(adv[0], torch.full((2,), 3.0))
    m = _lm(2)
    tokens = torch.randint(0, 50, (8, 10))
    mask = torch.ones(8, 10)
    with torch.no_grad():
        old = torch.log_softmax(m(tokens[:, :-1]).float(), -1).gather(-1, tokens[:, 1:, None]).squeeze(-1)
    g = GRPO(m, group=4)
    stats, aux = g.loss(None, {"tokens": tokens, "mask": mask, "rewards": torch.randn(8), "old_logprobs": old}, dew.Step())
    assert torch.isfinite(stats.total) and float(aux.metrics["clip_fraction"].value()) == 0.0

    class WithValue(nn.Module):
        def __init__(self, lm):
            super().__init__(); self.lm = lm; self.v = nn.Linear(50, 1)

        def forward(self, t):
            lg = self.lm(t)
            return lg, self.v(lg.float())
    p = PPO(WithValue(m), entropy_coef=0.01)
    stats, aux = p.loss(None, {"tokens": tokens, "mask": mask, "advantages": torch.randn(8, 9), "returns": torch.randn(8, 9), "old_logprobs": old}, dew.Step())
    assert torch.isfinite(stats.total) and float(aux.metrics["entropy"].value()) > 0


def test_distillation_pulls_student_to_teacher():
    teacher, student = _lm(3), _lm(4)
    obj = Distillation(student, teacher)
    tokens = torch.randint(0, 50, (8, 12))
    tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=1e-2, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    tr.fit(dew.Loader(lambda part: iter([{"tokens": tokens}] * 40), batch=8), steps=30, log_every=10)
    assert t.rows[-1]["teacher_kl"] < t.rows[0]["teacher_kl"]


def test_placement_report_for_a_target_machine():
    model = CausalTransformer(vocab_size=1024, emb_features=256, num_layers=2, num_heads=8, num_kv_heads=4, mlp_features=512, max_seq_len=64,
                              device="meta")
    rep = placement_report(model, MeshSpec(fsdp=4, tensor=2), Layout(), devices=8, memory_bytes=180e9)
    assert rep["fits"] and rep["mesh"]["fsdp"] == 4 and rep["mesh"]["tensor"] == 2 and not rep["refusals"]
    qkv = next(l for l in rep["leaves"] if l["name"].endswith("layers.0.mixer.qkv_proj.weight"))
    assert qkv["shard_factor"] == 8
    bad = placement_report(model, MeshSpec(tensor=3), Layout(), devices=3)
    assert bad["refusals"]
    tiny = placement_report(model, MeshSpec(), Layout(), devices=1, memory_bytes=1e6)
    assert not tiny["fits"]
