"""Objectives beyond diffusion / LM: supervised, JEPA, DPO, GRPO, PPO, distillation; placement report."""
import pytest
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


def test_policy_update_rules_agree_on_policy_and_differ_off_policy():
    """On policy (the sampling weights are the trained ones) every update rule's gradient is REINFORCE's; off policy the clips,
    the sequence ratio and the sampler corrections change it."""
    torch.manual_seed(0)
    m = _lm(5)
    tokens = torch.randint(0, 50, (8, 10))
    mask = torch.ones(8, 10)
    mask[:, :3] = 0
    with torch.no_grad():
        old = torch.log_softmax(m(tokens[:, :-1]).float(), -1).gather(-1, tokens[:, 1:, None]).squeeze(-1)
    rewards = torch.randn(8)
    batch = {"tokens": tokens, "mask": mask, "rewards": rewards, "old_logprobs": old}

    def grad(obj, b=batch):
        m.zero_grad()
        stats, aux = obj.loss(None, b, dew.Step())
        (stats.total / stats.mass).backward()
        return torch.cat([p.grad.flatten() for p in m.parameters() if p.grad is not None]), aux

    base, _ = grad(GRPO(m, group=4, kl=0.0, rule="reinforce"))
    for rule in ("ppo", "cispo"):
        g, _ = grad(GRPO(m, group=4, kl=0.0, rule=rule, dual_clip=3.0 if rule == "ppo" else None))
        assert torch.allclose(g, base, atol=1e-5), rule
    gs, _ = grad(GRPO(m, group=4, kl=0.0, rule="gspo"))
    rs, _ = grad(GRPO(m, group=4, kl=0.0, rule="reinforce", reduction="seq-mean-token-mean"))
    assert torch.allclose(gs, rs, atol=1e-5)
    gm, _ = grad(GRPO(m, group=4, kl=0.0, rule="gmpo"))
    assert torch.isfinite(gm).all() and float(gm.norm()) > 0
    # estimators: leave-one-out is the centred reward times g / (g - 1); Dr. GRPO drops the deviation and normalises by the row length
    lo, _ = grad(GRPO(m, group=4, kl=0.0, rule="reinforce", advantage="rloo"))
    dr, _ = grad(GRPO(m, group=4, kl=0.0, rule="reinforce", advantage="dr_grpo", reduction="token-mean"))
    assert torch.allclose(lo, dr * 4 / 3, atol=1e-5)
    # off policy: a sampler far from the trainer is cut by the truncated weights, and a rejected sequence contributes nothing
    shifted = {**batch, "old_logprobs": old + 0.5, "behavior_logprobs": old + 0.5 + torch.tensor([3.0] * 4 + [0.0] * 4)[:, None]}
    plain, _ = grad(GRPO(m, group=4, kl=0.0), shifted)
    tis, aux = grad(GRPO(m, group=4, kl=0.0, importance="truncated"), shifted)
    rej, _ = grad(GRPO(m, group=4, kl=0.0, importance="reject", band=(0.5, 2.0)), shifted)
    assert not torch.allclose(plain, tis) and not torch.allclose(plain, rej) and "mismatch_k3_kl" in aux.metrics
    assert float(aux.metrics["clip_fraction"].value()) > 0
    with pytest.raises(ValueError):
        GRPO(m, rule="trpo")

    class WithValue(nn.Module):
        def __init__(self, lm):
            super().__init__(); self.lm = lm; self.v = nn.Linear(50, 1)

        def forward(self, t):
            lg = self.lm(t)
            return lg, self.v(lg.float())
    p = PPO(WithValue(m), value_clip=0.2, dual_clip=3.0, gamma=1.0, lam=0.95)
    stats, aux = p.loss(None, {"tokens": tokens, "mask": mask, "old_logprobs": old, "token_rewards": torch.randn(8, 9) * mask[:, 1:],
                               "old_values": torch.randn(8, 9)}, dew.Step())
    assert torch.isfinite(stats.total) and float(aux.metrics["value_loss"].value()) > 0


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


def test_masked_and_block_diffusion_lm_train_and_sample():
    from dew_b200.objectives.discrete import BlockDiffusionLM, MaskedDiffusionLM
    torch.manual_seed(0)
    V = 20
    class Bidirectional(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(V + 1, 32)
            self.mix = torch.nn.GRU(32, 32, batch_first=True, bidirectional=True)
            self.out = torch.nn.Linear(64, V + 1)
        def forward(self, tokens):
            return self.out(self.mix(self.emb(tokens))[0])
    data = (torch.arange(12)[None] + torch.arange(16)[:, None]) % V            # rows are arithmetic progressions
    for cls, kw in ((MaskedDiffusionLM, {}), (BlockDiffusionLM, {"block": 4})):
        obj = cls(Bidirectional(), mask_id=V, **kw)
        tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=1e-2, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
        st = tr.fit(dew.Memory({"tokens": data}).repeat().batched(16), steps=60, log_every=20)
        assert t.rows[-1]["masked_ce"] < t.rows[0]["masked_ce"]
        x = obj.sample(st.variables, 3, 12, steps=6, generator=torch.Generator().manual_seed(0))
        assert x.shape == (3, 12) and int((x == V).sum()) == 0
    assert BlockDiffusionLM.block_causal_mask(6, 2).tolist()[2] == [True, True, True, True, False, False]


def test_consistency_and_world_model_objectives():
    from dew_b200.objectives.consistency import ConsistencyObjective, WorldModelObjective
    torch.manual_seed(0)
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.f = torch.nn.Sequential(torch.nn.Linear(5, 32), torch.nn.SiLU(), torch.nn.Linear(32, 4))
        def forward(self, x, t):
            return self.f(torch.cat([x, t[:, None]], -1))
    obj = ConsistencyObjective(Net(), levels=8, ema_decay=0.9)
    # boundary condition: at sigma_min the denoiser is the identity
    x = torch.randn(3, 4)
    assert torch.allclose(obj.denoise(None, x, torch.full((3,), obj.smin)), x, atol=1e-5)
    tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=2e-3, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    st = tr.fit(dew.Memory({"sample": torch.randn(64, 4) * 0.5}).repeat().batched(16), steps=30, log_every=10)
    assert obj.generate(st.averaged, (5, 4), steps=2).shape == (5, 4) and all(r["loss"] == r["loss"] for r in t.rows)

    class World(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.enc, self.dyn = torch.nn.Linear(6, 8), torch.nn.Linear(8 + 2, 8)
            self.rew, self.don = torch.nn.Linear(8 + 2, 1), torch.nn.Linear(8, 1)
        def encode(self, o): return self.enc(o)
        def dynamics(self, z, a): return self.dyn(torch.cat([z, a], -1))
        def reward(self, z, a): return self.rew(torch.cat([z, a], -1))
        def done(self, z): return self.don(z)
    batch = {"observation": torch.randn(8, 5, 6), "action": torch.randn(8, 4, 2), "reward": torch.randn(8, 4), "done": torch.zeros(8, 4)}
    wobj = WorldModelObjective(World(), horizon=3)
    tr = dew.Trainer(wobj, dew.OptimConfig(learning_rate=1e-2, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    tr.fit(dew.Loader(lambda part: iter([batch] * 30), batch=8), steps=20, log_every=5)
    assert t.rows[-1]["loss"] < t.rows[0]["loss"]


def test_multi_token_prediction_heads_train():
    """MTP depths add their cross-entropy (weighted) to the loss, report their own metrics and receive gradients."""
    import torch
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.base import Step
    from dew_b200.objectives.lm import LMObjective
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=50, emb_features=32, num_layers=2, num_heads=4, head_dim=8, mlp_features=64, max_seq_len=32,
                              mtp_depth=2)
    plain = LMObjective(model, 16)
    mtp = LMObjective(model, 16, mtp_weight=0.3)
    batch = {"tokens": torch.randint(0, 50, (3, 17))}
    s0, _ = plain.loss(None, batch, Step(train=True))
    s1, aux = mtp.loss(None, batch, Step(train=True))
    l0, l1 = float(s0.value()), float(s1.value())
    assert l1 > l0 and "mtp_loss_1" in aux.metrics and "mtp_loss_2" in aux.metrics
    want = l0 + 0.3 * 0.5 * (float(aux.metrics["mtp_loss_1"].value()) + float(aux.metrics["mtp_loss_2"].value()))
    assert abs(l1 - want) < 1e-4
    s1.value().backward()
    assert model.mtp[1].proj.weight.grad.abs().sum() > 0
    hs = model.mtp_hiddens(model(batch["tokens"][:, :-1], return_hidden=True), batch["tokens"])
    assert [h.shape[1] for h in hs] == [15, 14]


class _TimeNet(torch.nn.Module):
    """A small velocity network ``(x [rows, d], t [rows], extra [rows]) -> [rows, d]``."""

    def __init__(self, d=6, extra=True):
        super().__init__()
        self.net = torch.nn.Sequential(torch.nn.Linear(d + (2 if extra else 1), 32), torch.nn.SiLU(), torch.nn.Linear(32, d))
        self.extra = extra

    def forward(self, x, t, r=None, **kw):
        cols = [x, t[:, None]] + ([r[:, None]] if self.extra else [])
        return self.net(torch.cat(cols, -1))


def test_meanflow_and_shortcut_objectives_learn_a_point_mass():
    """Both few-step objectives pull a one-step sample towards the data (a point mass at 2) and their losses fall."""
    from dew_b200.objectives.base import Step
    from dew_b200.objectives.few_step import MeanFlowObjective, ShortcutObjective
    for cls in (MeanFlowObjective, ShortcutObjective):
        torch.manual_seed(0)
        model = _TimeNet()
        obj = cls(model)
        opt = torch.optim.Adam(model.parameters(), lr=3e-3)
        data = {"sample": torch.full((64, 6), 2.0)}
        first = last = None
        for i in range(150):
            stats, _ = obj.loss(None, data, Step(train=True, key=i))
            loss = stats.value()
            opt.zero_grad(); loss.backward(); opt.step()
            first = float(loss) if first is None else first
            last = float(loss)
        assert last < first
        out = obj.generate(None, (256, 6), generator=torch.Generator().manual_seed(1), steps=1)
        assert abs(float(out.mean()) - 2.0) < 0.5, (cls.__name__, float(out.mean()))


def test_flow_grpo_raises_the_reward():
    from dew_b200.objectives.base import Step
    from dew_b200.objectives.rl.policy import FlowGRPO
    torch.manual_seed(0)
    model = _TimeNet(d=4, extra=False)
    obj = FlowGRPO(model, group=8, noise_level=0.5)
    opt = torch.optim.Adam(model.parameters(), lr=2e-3)
    reward = lambda x: -(x - 1.0).pow(2).mean(-1)              # prefers samples near 1
    means = []
    for it in range(30):
        xs, grid, old = obj.rollout(None, (64, 4), steps=6, generator=torch.Generator().manual_seed(it))
        r = reward(xs[:, -1])
        means.append(float(r.mean()))
        if it == 0:                                            # the stored log-density is the policy's own
            lp, _ = obj.logp(None, xs[:, 0], xs[:, 1], grid[0], grid[0] - grid[1])
            assert torch.allclose(lp, old[:, 0], atol=1e-4)
        stats, aux = obj.loss(None, {"x": xs, "t": grid, "old_logp": old, "rewards": r}, Step(train=True, key=it))
        opt.zero_grad(); stats.value().backward(); opt.step()
    assert sum(means[-5:]) / 5 > sum(means[:5]) / 5


def test_fit_cooldown_summaries_loss_role_and_preview():
    import dew_b200 as dew
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=32, emb_features=32, num_layers=1, num_heads=4, head_dim=8, mlp_features=64, max_seq_len=16)
    obj = LMObjective(model, 8, loss_role=2, samples={"prompt": [1, 2, 3], "max_new_tokens": 4})
    tokens = torch.randint(0, 32, (16, 9))
    roles = torch.ones(16, 9, dtype=torch.long)
    roles[:, 5:] = 2
    assert obj.scored_tokens({"tokens": tokens, "roles": roles}) == 16 * 4        # only the role's targets are scored
    trainer = dew.Trainer(obj, dew.OptimConfig(learning_rate=1e-2), tracker=dew.MemoryTracker())
    state = trainer.fit(dew.Memory({"tokens": tokens, "roles": roles}).repeat().batched(8), steps=10, log_every=2,
                        cooldowns=[dew.Cooldown(at=4, steps=4, floor=0.1)], summaries=lambda st: {"updates": st.step})
    rates = [r["learning_rate"] for r in trainer.tracker.rows if "learning_rate" in r]
    assert rates[0] == pytest.approx(1e-2) and rates[-1] == pytest.approx(1e-3, rel=1e-3) and all("updates" in r for r in trainer.tracker.rows if "loss" in r)
    assert trainer.optimizer.schedule(9) == pytest.approx(1e-2)                    # the trunk schedule is back after the fit
    art = obj.preview(state.variables, key=0)
    assert len(art.completions) == 1 and len(art.completions[0].split()) == 4
    with pytest.raises(ValueError):
        LMObjective(model, 8, exit_entropy=0.1)                                    # no loop to gate
    with pytest.raises(NotImplementedError):
        LMObjective(model, 8, indexer=object())
    assert dew.Cooldown(0, 10, 0.0, "sqrt").factor(10) == 0.0 and dew.Cooldown(5, 10).factor(3) == 1.0


def test_looped_decoder_trains_its_passes_and_its_exit_gate():
    from dew_b200.models.causal_transformer import Loop
    from dew_b200.objectives.lm import LMObjective
    torch.manual_seed(0)
    mk = lambda **kw: CausalTransformer(vocab_size=24, emb_features=32, num_layers=3, num_heads=2, head_dim=16, mlp_features=64, max_seq_len=16,
                                        qk_norm=False, loop=Loop(steps=3, first=1, end=2, **kw))
    tokens = torch.randint(0, 24, (16, 9))
    model = mk(exit_gate=True)
    outs = model(tokens[:, :-1], passes=True)
    assert len(outs) == 3 and torch.allclose(model(tokens[:, :-1]), outs[-1]) and torch.allclose(model(tokens[:, :-1], loop_steps=2), outs[1])
    p = model.exit_distribution(model(tokens[:, :-1], return_hidden=True, passes=True))
    assert p.shape == (3, 16, 8) and torch.allclose(p.sum(0), torch.ones(16, 8), atol=1e-6)
    # the exit objective: expected cross entropy under the exit distribution less beta times its entropy
    obj = LMObjective(model, 8, exit_entropy=0.05)
    stats, aux = obj.loss(None, {"tokens": tokens}, dew.Step(train=True))
    m = {k: float(v.value()) for k, v in aux.metrics.items()}
    assert float(stats.value()) == pytest.approx(m["exit_ce"] - 0.05 * m["exit_entropy"], rel=1e-5) and 1.0 <= m["exit_depth"] <= 3.0
    stats.value().backward()
    assert model.early_exit_gate.weight.grad is not None and float(model.early_exit_gate.weight.grad.abs().sum()) > 0
    # pass weights: each pass's own cross entropy, weighed; all weight on the last pass is the plain objective
    plain = mk()
    last_only = LMObjective(plain, 8, pass_weights=(0.0, 0.0, 1.0))
    a, _ = last_only.loss(None, {"tokens": tokens}, dew.Step(train=True))
    b, _ = LMObjective(plain, 8).loss(None, {"tokens": tokens}, dew.Step(train=True))
    assert float(a.value()) == pytest.approx(float(b.value()), rel=1e-4)
    mean = LMObjective(plain, 8, pass_weights="mean")
    st, aux = mean.loss(None, {"tokens": tokens}, dew.Step(train=True))
    per = [float(aux.metrics[f"pass_{i}_ce"].value()) for i in (1, 2, 3)]
    assert float(st.value()) == pytest.approx(sum(per) / 3, rel=1e-5)
    tr = dew.Trainer(mean, dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    tr.fit([{"tokens": tokens}] * 40, steps=40, log_every=10)
    assert t.rows[-1]["pass_1_ce"] < 0.8 * per[0] and t.rows[-1]["loss"] < t.rows[0]["loss"]          # every pass count learns
    # the passes before the last backprop_steps carry no gradient
    cut = mk(backprop_steps=1)
    LMObjective(cut, 8).loss(None, {"tokens": tokens}, dew.Step(train=True))[0].value().backward()
    assert cut.layers[0].mlp.gate_up_proj.weight.grad is None and cut.layers[1].mlp.gate_up_proj.weight.grad is not None
    with pytest.raises(ValueError):
        LMObjective(plain, 8, pass_weights=(0.5, 0.5))
    with pytest.raises(ValueError):
        LMObjective(model, 8, exit_entropy=0.1, pass_weights="mean")
    with pytest.raises(NotImplementedError):
        from dew_b200.nn.kv_cache import KVCache, KVStore
        model(tokens[:, :-1], cache=object())
    with pytest.raises(ValueError):
        Loop(steps=2, backprop_steps=3)


def test_node_perturbation_estimates_the_gradient_and_trains_without_backprop():
    import torch
    import dew_b200 as dew
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives import Step
    from dew_b200.objectives.lm import LMObjective
    from dew_b200.objectives.perturbation import NodePerturbation
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=32, emb_features=32, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=48, max_seq_len=16,
                              tie_embeddings=False)
    tokens = torch.randint(0, 32, (8, 17))
    # the true gradient of the head
    model.zero_grad()
    stat, _ = LMObjective(model, 16, ema_decay=None).loss(None, {"tokens": tokens}, Step(key=0, train=True))
    (stat.total / stat.mass).backward()
    true = model.head.weight.grad.clone()
    est = torch.zeros_like(true)
    obj = NodePerturbation(model, 16, sigma=1e-2, draws=16)
    for k in range(8):
        model.zero_grad()
        s, aux = obj.loss(None, {"tokens": tokens}, Step(key=k, train=True))
        assert abs(float(s.total / s.mass) - float(stat.total / stat.mass)) < 1e-4          # the value is the clean loss
        (s.total / s.mass).backward()
        est += model.head.weight.grad
    cos = float((est * true).sum() / (est.norm() * true.norm()))
    assert cos > 0.15, cos                     # a noisy but aligned estimate (every node is jittered at once)
    # a few hundred forward-only steps lower the loss on a fixed batch
    trainer = dew.Trainer(NodePerturbation(model, 16, sigma=1e-2, draws=4), dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0), key=0,
                          tracker=dew.MemoryTracker())
    trainer.fit([{"tokens": tokens}] * 120, steps=120, log_every=20)
    losses = [r["loss"] for r in trainer.tracker.rows if "loss" in r]
    assert losses[-1] < losses[0] - 0.1, losses


def test_adaptive_lm_objective_steps_a_level_in_context():
    import torch
    import dew_b200 as dew
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives import Step
    from dew_b200.objectives.adaptation import AdaptiveLMObjective, ChunkAdaptation, Continuum
    from dew_b200.objectives.lm import LMObjective
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=32, emb_features=32, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=48, max_seq_len=32,
                              tie_embeddings=False)
    tokens = torch.randint(0, 32, (3, 33))
    plain, _ = LMObjective(model, 32, ema_decay=None).loss(None, {"tokens": tokens}, Step(key=0, train=True))
    # the level starts as the identity, and a single window takes no step: the loss is the model's own
    obj = AdaptiveLMObjective(model, 32, ChunkAdaptation(window=32, rate=0.1))
    one, aux = obj.loss(None, {"tokens": tokens}, Step(key=0, train=True))
    assert torch.allclose(one.total / one.mass, plain.total / plain.mass, atol=1e-5) and float(aux.metrics["level_step"].value()) == 0.0
    # windows of 8: later windows read a stepped level, so the loss differs, and the start gets a (meta-)gradient
    obj8 = AdaptiveLMObjective(model, 32, ChunkAdaptation(window=8, rate=0.5))
    with torch.no_grad():
        obj8.model.continuum.up.normal_(0, 0.05)
    s8, a8 = obj8.loss(None, {"tokens": tokens}, Step(key=0, train=True))
    assert float(a8.metrics["level_step"].value()) > 0
    (s8.total / s8.mass).backward()
    assert obj8.model.continuum.down.grad is not None and float(obj8.model.continuum.down.grad.abs().sum()) > 0
    full = obj8.model.continuum.down.grad.clone()
    obj8.model.zero_grad()
    first = AdaptiveLMObjective(model, 32, ChunkAdaptation(window=8, rate=0.5, first_order=True))
    first.model.continuum.load_state_dict(obj8.model.continuum.state_dict())
    sf, _ = first.loss(None, {"tokens": tokens}, Step(key=0, train=True))
    assert torch.allclose(sf.total, s8.total, atol=1e-5)                       # same forward ...
    (sf.total / sf.mass).backward()
    assert not torch.allclose(first.model.continuum.down.grad, full, atol=1e-7)   # ... different gradient without the meta term
    # adapting in context helps on rows that repeat themselves: after training, the stepped level beats the frozen one
    rep = torch.randint(0, 32, (16, 8)).repeat(1, 5)[:, :33]
    trainer = dew.Trainer(obj8, dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0), key=0, tracker=dew.MemoryTracker())
    trainer.fit([{"tokens": rep}] * 40, steps=40, log_every=10)
    losses = [r["loss"] for r in trainer.tracker.rows if "loss" in r]
    assert losses[-1] < losses[0]
    lvl = Continuum(4, 6)
    x = torch.randn(2, 3, 4)
    assert torch.equal(lvl(x), x)
