"""Attention variants, the normalised transformer, vector quantisers and Fourier feature pyramids against direct formulas."""
import math

import pytest
import torch

from dew_b200.nn.attention_variants import (DifferentialAttention, ForgettingAttention, LightningIndexer, ValueExperts, biased_attention,
                                            block_sparse_attention, forgetting_bias, indexed_sparse_attention, indexer_alignment_loss, lambda_init,
                                            moba_selection, top_k_selection)
from dew_b200.nn.fourier import FourierFeaturePyramid, fourier_features
from dew_b200.nn.normalized import NormalizedBlock, Scale, justnorm, normalize_weights_, sphere_step
from dew_b200.nn.quantizers import FSQ, LFQ, ResidualVQ


def _dense(q, k, v, mask=None, bias=None):
    s = torch.einsum("bshd,bthd->bhst", q, k) * q.shape[-1] ** -0.5
    if bias is not None:
        s = s + bias
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("bhst,bthd->bshd", torch.softmax(s, -1), v)


def test_biased_attention_groups_heads_and_masks():
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 6, 4, 8), torch.randn(2, 6, 2, 8), torch.randn(2, 6, 2, 8)
    causal = torch.tril(torch.ones(6, 6, dtype=torch.bool))[None, None]
    full = _dense(q, k.repeat_interleave(2, 2), v.repeat_interleave(2, 2), causal)
    assert torch.allclose(biased_attention(q, k, v, mask=causal), full, atol=1e-5)
    none = torch.zeros(1, 1, 6, 6, dtype=torch.bool)
    assert torch.all(biased_attention(q, k, v, mask=none) == 0)             # a query that sees nothing returns zeros, not NaN


def test_differential_attention_is_the_difference_of_two_maps():
    torch.manual_seed(0)
    m = DifferentialAttention(32, num_heads=2, layer=3)
    assert m.lambda_init == pytest.approx(0.8 - 0.6 * math.exp(-0.9)) and lambda_init(0) == pytest.approx(0.2)
    x = torch.randn(2, 5, 32)
    out = m(x)
    d = m.head_dim
    q = m.q_proj(x).view(2, 5, 4, d); k = m.k_proj(x).view(2, 5, 4, d); v = m.v_proj(x).view(2, 5, 2, 2 * d)
    causal = torch.tril(torch.ones(5, 5, dtype=torch.bool))[None, None]
    maps = []
    for half in (0, 1):
        s = torch.einsum("bshd,bthd->bhst", q[:, :, half::2], k[:, :, half::2]) * d ** -0.5
        maps.append(torch.softmax(s.masked_fill(~causal, float("-inf")), -1))
    diff = torch.einsum("bhst,bthd->bshd", maps[0] - m.lam() * maps[1], v)
    want = m.o_proj((m.subln(diff) * (1 - m.lambda_init)).reshape(2, 5, -1))
    assert torch.allclose(out, want, atol=1e-5)
    out.sum().backward()
    assert m.lambda_q1.grad is not None and float(m.lambda_q1.grad.abs().sum()) > 0


def test_forgetting_attention_fades_keys_by_the_gates_between():
    lg = torch.log(torch.tensor([[[0.5], [0.25], [1.0], [0.5]]]))          # one head
    b = forgetting_bias(lg)[0, 0]
    assert torch.allclose(b[3, 0], torch.log(torch.tensor(0.25 * 1.0 * 0.5))) and torch.allclose(b[2, 2], torch.tensor(0.0))
    assert torch.allclose(b[3, 2], torch.log(torch.tensor(0.5)))
    torch.manual_seed(0)
    m = ForgettingAttention(32, num_heads=4, num_kv_heads=2)
    x = torch.randn(2, 7, 32)
    out = m(x)
    # with the gates forced open (f = 1) it is ordinary causal attention
    with torch.no_grad():
        m.gate_proj.weight.zero_(); m.gate_proj.bias.fill_(40.0)
    qkv = m.qkv_proj(x).view(2, 7, 8, 8)
    q, k, v = m.q_norm(qkv[:, :, :4]), m.k_norm(qkv[:, :, 4:6]), qkv[:, :, 6:]
    causal = torch.tril(torch.ones(7, 7, dtype=torch.bool))[None, None]
    plain = m.o_proj(_dense(q, k.repeat_interleave(2, 2), v.repeat_interleave(2, 2), causal).reshape(2, 7, 32))
    assert torch.allclose(m(x), plain, atol=1e-4) and not torch.allclose(out, plain, atol=1e-3)
    # closed gates (f -> 0): each query reads only itself
    with torch.no_grad():
        m.gate_proj.bias.fill_(-40.0)
    self_only = m.o_proj(v.repeat_interleave(2, 2).reshape(2, 7, 32))
    assert torch.allclose(m(x), self_only, atol=1e-4)


def test_block_selection_and_indexed_sparse_attention():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 16, 2, 8), torch.randn(1, 16, 1, 8), torch.randn(1, 16, 1, 8)
    sel = moba_selection(q, k, block=4, top_k=2)
    assert sel.shape == (1, 1, 16, 2) and sel[0, 0, :, 0].tolist() == [i // 4 for i in range(16)]
    assert torch.all(sel[0, 0, :4, 1] == -1) and torch.all(sel[0, 0, 4:8, 1] == 0)          # the first block has nothing earlier; the second only block 0
    assert torch.all((sel[0, 0, 8:, 1] >= 0) & (sel[0, 0, 8:, 1] < sel[0, 0, 8:, 0]))
    out = block_sparse_attention(q, k, v, sel, block=4)
    # selecting every earlier block is dense causal attention
    every = moba_selection(q, k, block=4, top_k=4)
    causal = torch.tril(torch.ones(16, 16, dtype=torch.bool))[None, None]
    dense = _dense(q, k.repeat_interleave(2, 2), v.repeat_interleave(2, 2), causal)
    assert torch.allclose(block_sparse_attention(q, k, v, every, block=4), dense, atol=1e-5) and not torch.allclose(out, dense, atol=1e-3)
    # the key with the dominant score is always selected by a top-1 index, and attending to it alone returns its value
    x = torch.randn(1, 10, 16)
    idx = LightningIndexer(16, heads=2, head_dim=8)
    scores = idx(x)
    assert scores.shape == (1, 10, 10)
    chosen = top_k_selection(scores, 3)
    assert chosen.shape == (1, 10, 3) and int((chosen[0, 0] >= 0).sum()) == 1 and torch.all(chosen[0, 5][chosen[0, 5] >= 0] <= 5)
    one = top_k_selection(scores, 1)
    qq, kk, vv = torch.randn(1, 10, 2, 8), torch.randn(1, 10, 1, 8), torch.randn(1, 10, 1, 8)
    got = indexed_sparse_attention(qq, kk, vv, one)
    assert torch.allclose(got[0, :, 0], vv[0, one[0, :, 0], 0], atol=1e-6)
    all_keys = top_k_selection(scores, 10)
    assert torch.allclose(indexed_sparse_attention(qq, kk, vv, all_keys), _dense(qq, kk.repeat_interleave(2, 2), vv.repeat_interleave(2, 2), torch.tril(torch.ones(10, 10, dtype=torch.bool))[None, None]), atol=1e-5)
    probs = torch.softmax(torch.randn(1, 2, 10, 10).masked_fill(~torch.tril(torch.ones(10, 10, dtype=torch.bool)), float("-inf")), -1)
    loss = indexer_alignment_loss(scores, probs)
    loss.backward()
    assert float(loss) > 0 and idx.q_proj.weight.grad is not None
    perfect = indexer_alignment_loss(torch.log(probs.sum(1).clamp_min(1e-30)), probs)
    assert float(perfect) < 1e-5


def test_value_experts_route_top_k():
    torch.manual_seed(0)
    m = ValueExperts(16, 8, experts=4, top_k=2)
    x = torch.randn(3, 5, 16)
    out = m(x)
    scores = torch.sigmoid(m.router(x))
    top = scores.topk(2, -1)
    w = top.values / top.values.sum(-1, keepdim=True)
    want = torch.zeros(3, 5, 8)
    for b in range(3):
        for t in range(5):
            for j in range(2):
                e = int(top.indices[b, t, j])
                want[b, t] += w[b, t, j] * torch.nn.functional.silu(m.weight[e] @ x[b, t])
    assert torch.allclose(out, want, atol=1e-5)
    m.balance_bias[:] = torch.tensor([100.0, 100.0, 0.0, 0.0])             # the bias changes who is chosen, not the weights' source
    biased = m(x)
    s01 = scores[..., :2] / scores[..., :2].sum(-1, keepdim=True)
    w0 = s01[..., 0:1] * torch.nn.functional.silu(torch.einsum("btf,of->bto", x, m.weight[0])) + s01[..., 1:2] * torch.nn.functional.silu(torch.einsum("btf,of->bto", x, m.weight[1]))
    assert torch.allclose(biased, w0, atol=1e-5)


def test_normalized_transformer_keeps_states_and_weights_on_the_sphere():
    torch.manual_seed(0)
    x = torch.randn(4, 16)
    assert torch.allclose(justnorm(x).norm(dim=-1), torch.ones(4), atol=1e-6)
    h, y = justnorm(torch.randn(2, 3, 16)), torch.randn(2, 3, 16)
    assert torch.allclose(sphere_step(h, y, torch.zeros(16)), h, atol=1e-6)
    assert torch.allclose(sphere_step(h, y, torch.ones(16)), justnorm(y), atol=1e-6)
    s = Scale(8, init=0.05, scale=8 ** -0.5)
    assert torch.allclose(s(), torch.full((8,), 0.05)) and float(s.value[0]) == pytest.approx(8 ** -0.5)
    block = NormalizedBlock(32, num_heads=4, hidden=64, layers=6)
    assert normalize_weights_(block) == 4
    assert torch.allclose(block.attn.qkv.weight.norm(dim=1), torch.ones(96), atol=1e-5) and torch.allclose(block.mlp.down.weight.norm(dim=0), torch.ones(64), atol=1e-5)
    hidden = justnorm(torch.randn(2, 9, 32))
    out = block(hidden)
    assert torch.allclose(out.norm(dim=-1), torch.ones(2, 9), atol=1e-5)
    # causal: changing a later token leaves earlier outputs alone
    other = hidden.clone(); other[:, 5:] = justnorm(torch.randn(2, 4, 32))
    assert torch.allclose(block(other)[:, :5], out[:, :5], atol=1e-5)
    opt = torch.optim.SGD(block.parameters(), lr=0.1)
    block(hidden).pow(3).sum().backward(); opt.step(); normalize_weights_(block)
    assert torch.allclose(block.attn.out.weight.norm(dim=0), torch.ones(32), atol=1e-5)


def test_quantizers():
    torch.manual_seed(0)
    rvq = ResidualVQ(4, sizes=(8, 8, 8))
    x = torch.randn(5, 7, 4)
    codes = rvq.encode(x)
    assert codes.shape == (5, 7, 3) and int(codes.max()) < 8
    # stage by stage: the nearest codeword to the residual
    r = x[0, 0].clone()
    for s, table in enumerate(rvq.codebooks):
        idx = int(((r[None] - table) ** 2).sum(-1).argmin())
        assert idx == int(codes[0, 0, s])
        r = r - table[idx]
    assert torch.allclose(rvq.decode(codes)[0, 0], x[0, 0] - r.detach(), atol=1e-5)
    xq = x.clone().requires_grad_()
    q, c2, loss = rvq(xq)
    assert torch.equal(c2, codes) and torch.allclose(q, rvq.decode(codes), atol=1e-5)
    (q.sum() + loss).backward()
    assert xq.grad is not None and rvq.codebooks[0].grad is not None
    fsq = FSQ((8, 5, 5))
    assert fsq.codebook_size == 200
    z = torch.randn(1000, 3) * 3
    zq, idx = fsq(z)
    assert float(zq.abs().max()) <= 1.0 + 1e-6 and int(idx.max()) < 200 and int(idx.min()) >= 0 and len(idx.unique()) > 100
    assert torch.allclose(fsq.decode(idx), zq, atol=1e-5)
    assert len(zq[:, 1].unique()) == 5 and len(zq[:, 0].unique()) == 8
    zz = z.clone().requires_grad_()
    fsq(zz)[0].sum().backward()
    assert float(zz.grad.abs().sum()) > 0                                  # straight through the rounding
    lfq = LFQ(bits=6)
    zb = torch.randn(256, 6)
    qb, cb, lb = lfq(zb)
    assert set(qb.unique().tolist()) == {-1.0, 1.0} and int(cb.max()) < 64 and torch.isfinite(lb)
    assert torch.equal(cb, ((zb > 0).long() * 2 ** torch.arange(6)).sum(-1))
    collapsed = lfq(torch.ones(256, 6) * 3)[2]
    assert float(collapsed) > float(lb)                                    # one code for the whole batch is penalised


def test_fourier_pyramid_interpolates_its_grids_and_differentiates():
    torch.manual_seed(0)
    for n in (4, 5):
        pyr = FourierFeaturePyramid(dims=2, features=3, resolutions=(n,), init=1.0)
        pts = torch.stack(torch.meshgrid(torch.arange(n) / n, torch.arange(n) / n, indexing="ij"), -1).reshape(-1, 2)
        got = pyr(pts).reshape(n, n, 3).permute(2, 0, 1)
        assert torch.allclose(got, pyr.grids[0], atol=1e-4), n                # exact at the grid points
    pyr = FourierFeaturePyramid(dims=1, features=2, resolutions=(4, 8))
    x = torch.rand(16, 1)
    assert pyr(x).shape == (16, 4) and torch.allclose(pyr(x), pyr(x + 1.0), atol=1e-4)          # periodic
    # a grid holding one cosine wave is read back as that wave everywhere, and its derivative is the wave's
    single = FourierFeaturePyramid(dims=1, features=1, resolutions=(8,))
    with torch.no_grad():
        single.grids[0].copy_(torch.cos(2 * math.pi * torch.arange(8) / 8)[None])
    xs = torch.rand(20, 1, requires_grad=True)
    ys = single(xs)
    assert torch.allclose(ys[:, 0], torch.cos(2 * math.pi * xs[:, 0]), atol=1e-4)
    (dy,) = torch.autograd.grad(ys.sum(), xs, create_graph=True)
    assert torch.allclose(dy[:, 0], -2 * math.pi * torch.sin(2 * math.pi * xs[:, 0]), atol=1e-3)
    (d2,) = torch.autograd.grad(dy.sum(), xs)
    assert torch.allclose(d2[:, 0], -(2 * math.pi) ** 2 * torch.cos(2 * math.pi * xs[:, 0]), atol=1e-2)
    assert fourier_features(torch.rand(5, 2), torch.randn(2, 7)).shape == (5, 14)
    with pytest.raises(ValueError):
        FourierFeaturePyramid(dims=4)


def test_variant_mixers_train_inside_the_decoder():
    from dew_b200.models import CausalTransformer
    torch.manual_seed(0)
    tokens = torch.randint(0, 32, (4, 12))
    for kinds in (("differential",), ("forgetting", "attention")):
        m = CausalTransformer(vocab_size=32, emb_features=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=64, max_seq_len=16,
                              layer_types=kinds, qk_norm=False)
        logits = m(tokens)
        assert logits.shape == (4, 12, 32)
        # causal: a later token does not change earlier logits
        other = tokens.clone(); other[:, 8:] = (other[:, 8:] + 1) % 32
        assert torch.allclose(m(other)[:, :8], logits[:, :8], atol=1e-5), kinds
        loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 32).float(), tokens[:, 1:].reshape(-1))
        loss.backward()
        assert all(p.grad is not None for n, p in m.named_parameters() if "mixer" in n), kinds
