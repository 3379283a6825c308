"""The router policy (balancing bias, expert-level balance loss, router z-loss) on a tiny MoE decoder."""
import pytest
import torch

from dew_b200.models import CausalTransformer
from dew_b200.models.causal_transformer import Mixture
from dew_b200.objectives import Step
from dew_b200.objectives.lm import LMObjective
from dew_b200.objectives.routing import ExpertBalance, UntrainedRouter, refuse_fixed_routers, router_balance_loss


def _model(bias=True):
    return CausalTransformer(vocab_size=64, emb_features=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=48,
                             max_seq_len=16, qk_norm=False, tie_embeddings=False,
                             mixture=Mixture(experts=4, top_k=2, bias=bias, expert_features=24))


def test_balance_loss_forms():
    T, E, K = 12, 4, 2
    scores = torch.softmax(torch.randn(T, E), -1)
    ids = scores.topk(K, -1).indices
    whole = router_balance_loss(scores, ids, E)
    f = torch.bincount(ids.reshape(-1), minlength=E).float() * E / (K * T)
    assert torch.allclose(whole, (f * scores.mean(0)).sum(), atol=1e-6)
    # perfectly uniform routing scores 1
    uni = torch.full((8, E), 1.0 / E)
    uid = torch.tensor([[0, 1], [2, 3]] * 4)
    assert abs(float(router_balance_loss(uni, uid, E)) - 1.0) < 1e-6
    # per sequence: the mean of each sequence's own loss; padding (-1) is left out
    seq = torch.tensor([0] * 5 + [1] * 5 + [-1] * 2)
    per = router_balance_loss(scores, ids, E, seq)
    a = router_balance_loss(scores[:5], ids[:5], E)
    b = router_balance_loss(scores[5:10], ids[5:10], E)
    assert torch.allclose(per, (a + b) / 2, atol=1e-6)


def test_policy_terms_add_to_the_loss_and_move_the_bias():
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (3, 17))
    plain = LMObjective(_model(), 16, ema_decay=None)
    v = plain.init(0)
    base, _ = plain.loss(v, {"tokens": tokens}, Step(key=0, train=True))
    policy = ExpertBalance(balance_rate=1e-2, aux_loss_alpha=0.01, seq_aux=True, router_z_loss=1e-3)
    obj = LMObjective(_model(), 16, ema_decay=None, balance=policy)
    v2 = obj.init(0)
    stat, aux = obj.loss(v2, {"tokens": tokens}, Step(key=0, train=True))
    bal, z = aux.metrics["router_balance_loss"].value(), aux.metrics["router_z_loss"].value()
    assert float(bal) > 0 and float(z) > 0
    assert torch.allclose(stat.total / stat.mass, base.total / base.mass + 0.01 * bal + 1e-3 * z, atol=1e-5)
    # the terms reach the routers' weights
    (stat.total / stat.mass).backward()
    g = obj.model.layers[0].mlp.router.weight.grad
    assert g is not None and float(g.abs().sum()) > 0
    # effects: one bias update per sparse layer, by the policy's own rate, against the load
    assert sorted(aux.effects) == ["layers.0.mlp.router.expert_bias", "layers.1.mlp.router.expert_bias"]
    upd = aux.effects["layers.0.mlp.router.expert_bias"]
    assert all(abs(x) < 1e-9 or abs(x - 1e-2) < 1e-7 for x in upd.abs().tolist())
    obj.apply_effects(v2, aux.effects)
    assert torch.equal(obj.model.layers[0].mlp.router.expert_bias, upd)


def test_refusals():
    with pytest.raises(ValueError):
        ExpertBalance(balance_rate=0.0)
    with pytest.raises(ValueError):
        ExpertBalance(aux_loss_alpha=-1.0)
    with pytest.raises(UntrainedRouter):
        ExpertBalance(balance_rate=1e-3).prepare(_model(bias=False))
    dense = CausalTransformer(vocab_size=64, emb_features=32, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=48, max_seq_len=16)
    with pytest.raises(ValueError):
        ExpertBalance(aux_loss_alpha=0.01).prepare(dense)
    m = _model(bias=True)
    for layer in m.layers:
        layer.mlp.router.weight.requires_grad_(False)
    with pytest.raises(UntrainedRouter):
        refuse_fixed_routers(m, None)
    refuse_fixed_routers(m, ExpertBalance(balance_rate=1e-3))          # the bias still moves their choices
