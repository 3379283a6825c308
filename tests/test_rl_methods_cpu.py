"""The named RL methods build the objective their papers state, and DAPO's batch steps."""
import pytest
import torch

from dew_b200.objectives.base import Step
from dew_b200.objectives.rl.methods import METHODS, method, overlong_punishment, prepare, reward_with_reference, varied_groups
from dew_b200.rl.advantage import global_advantage


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = torch.nn.Embedding(11, 8)
        self.out = torch.nn.Linear(8, 11)

    def forward(self, tokens):
        return self.out(self.emb(tokens))


def test_table_and_free_settings():
    model = Tiny()
    assert sorted(METHODS) == ["cispo", "dapo", "dr_grpo", "gmpo", "grpo", "gspo", "reinforce_pp", "rloo"]
    dapo = method("dapo", model, group=4)
    assert (dapo.clip, dapo.clip_high, dapo.kl, dapo.reduction) == (0.2, 0.28, 0.0, "token-mean")
    grpo = method("grpo", model, group=4, beta=0.1)
    assert grpo.kl == 0.1 and grpo.kl_kind == "k3" and grpo.rule == "ppo"
    assert method("reinforce_pp", model).advantage == "global" and method("reinforce_pp", model).kl_kind == "k2"
    rloo = method("rloo", model, reward_kl=0.05)
    assert rloo.rule == "reinforce" and rloo.reward_kl == 0.05 and rloo.kl == 0.0
    assert method("gspo", model, clip=1e-3, clip_high=2e-3).clip_high == 2e-3
    with pytest.raises(ValueError, match="fixes"):
        method("dapo", model, beta=0.1)
    with pytest.raises(KeyError, match="known"):
        method("ppo2", model)


def test_every_method_gives_a_finite_loss_and_gradient():
    torch.manual_seed(0)
    model = Tiny()
    tokens = torch.randint(0, 11, (8, 7))
    mask = torch.zeros(8, 7)
    mask[:, 3:] = 1
    with torch.no_grad():
        old = torch.log_softmax(model(tokens[:, :-1]), -1).gather(-1, tokens[:, 1:, None]).squeeze(-1) + 0.05 * torch.randn(8, 6)
    batch = {"tokens": tokens, "mask": mask, "rewards": torch.randn(8), "old_logprobs": old}
    for name in METHODS:
        obj = method(name, model, group=4)
        stats, _ = obj.loss(None, batch, Step(step=0))
        value = stats.total / stats.mass
        assert torch.isfinite(value), name
        grads = torch.autograd.grad(value, list(model.parameters()), allow_unused=True)
        assert any(g is not None and float(g.abs().sum()) > 0 for g in grads), name


def test_batch_steps():
    r = torch.tensor([1.0, 1.0, 0.0, 1.0, 0.0, 0.0])
    batch = {"rewards": r, "tokens": torch.arange(12).view(6, 2), "note": "kept as it is"}
    out, kept = varied_groups(batch, group=2)
    assert out["rewards"].tolist() == [0.0, 1.0] and out["tokens"].tolist() == [[4, 5], [6, 7]] and kept == pytest.approx(1 / 3) and out["note"] == "kept as it is"
    pen = overlong_punishment(torch.tensor([10, 80, 90, 100, 130]), limit=100, buffer=20)
    assert torch.allclose(pen, torch.tensor([0.0, 0.0, -0.5, -1.0, -1.0]))
    lp, ref = torch.tensor([[-1.0, -1.0, -1.0]]), torch.tensor([[-1.5, -1.0, -3.0]])
    assert reward_with_reference(torch.tensor([2.0]), lp, ref, torch.tensor([[1.0, 1.0, 0.0]]), 0.1).item() == pytest.approx(2.0 - 0.1 * 0.5)
    a = global_advantage(torch.tensor([1.0, 0.0, 10.0, 0.0]), 2)
    assert torch.allclose(a[:2] * 10, a[2:], atol=1e-5) and abs(float(a.mean())) < 1e-6      # one scale for every group
    model = Tiny()
    dapo = method("dapo", model, group=2)
    mask = torch.zeros(6, 9)
    mask[:, 2:] = 1
    mask[0, 6:] = 0
    prepared, report = prepare(dapo, {"rewards": r.clone(), "mask": mask, "tokens": torch.zeros(6, 9, dtype=torch.long), "old_logprobs": torch.zeros(6, 8)},
                               limit=7, buffer=2)
    assert report["overlong_share"] == pytest.approx(5 / 6) and report["groups_kept"] == pytest.approx(2 / 3)
    assert prepared["rewards"].shape[0] == 4
