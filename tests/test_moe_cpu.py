"""Mixture-of-experts bookkeeping on CPU: aligned expert-sorted layout, grouped products, capacity, balancing."""
import torch

from dew_b200.models.causal_transformer import CausalTransformer, Mixture
from dew_b200.nn.moe import capacity_positions, load_balance_update
from dew_b200.ops import grouped as G


def test_group_layout_is_aligned_and_complete():
    torch.manual_seed(0)
    T, k, E = 77, 3, 5
    ids = torch.randint(0, E, (T, k))
    lay = G.group_layout(ids, E)
    off = lay.offsets.tolist()
    assert all(o % 128 == 0 for o in off)
    assert lay.positions.unique().numel() == T * k                 # a bijection into the padded buffer
    flat = ids.reshape(-1)
    for g in range(E):
        pos = lay.positions[flat == g]
        assert ((pos >= off[g]) & (pos < off[g] + int(lay.counts[g]))).all()
    tiles = lay.tile_group.tolist()
    for t, g in enumerate(tiles):
        if g >= 0:
            assert off[g] <= t * 128 < off[g + 1]


def test_grouped_linear_matches_dense_loop_and_combines():
    torch.manual_seed(1)
    T, k, E, d, F = 40, 2, 4, 16, 24
    ids = torch.randint(0, E, (T, k))
    lay = G.group_layout(ids, E)
    x = torch.randn(T, d)
    w = torch.randn(E, F, d, requires_grad=True)
    weights = torch.rand(T, k)
    y = G.combine(G.grouped_linear(G.permute(x, lay, k), w, lay), lay, weights, T)
    ref = torch.zeros(T, F)
    for t in range(T):
        for j in range(k):
            ref[t] += weights[t, j] * (x[t] @ w[ids[t, j]].t())
    assert torch.allclose(y, ref, atol=1e-4)
    y.sum().backward()
    (gref,) = torch.autograd.grad(ref.sum(), w)
    assert torch.allclose(w.grad, gref, atol=1e-4)


def test_capacity_and_balance_update():
    ids = torch.tensor([[0], [0], [0], [1]])
    keep = capacity_positions(ids, 2, capacity=2)
    assert keep.reshape(-1).tolist() == [True, True, False, True]
    bias = load_balance_update(torch.zeros(3), torch.tensor([10, 1, 4]), 0.1)
    assert bias.tolist() == [-0.10000000149011612, 0.10000000149011612, 0.10000000149011612]


def test_moe_transformer_trains_and_reports_balance():
    torch.manual_seed(0)
    m = CausalTransformer(vocab_size=64, emb_features=32, num_layers=2, num_heads=4, mlp_features=64, max_seq_len=32,
                          mixture=Mixture(experts=4, top_k=2, expert_features=16, shared_features=32, bias=True))
    out = m(torch.randint(0, 64, (2, 16)))
    out.float().logsumexp(-1).sum().backward()
    aux = m.pop_aux()
    assert "balance_loss" in aux and len(aux["effects"]) == 2
    assert m.layers[0].mlp.experts.gate_up.grad.abs().sum() > 0
    assert m.param_count(active=True) < m.param_count()
