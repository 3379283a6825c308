"""DEX (a learned differential on chosen heads of a pretrained attention layer) and block attention residuals (the residual as a softmax over depth)."""
import pytest
import torch

from dew_b200.models.causal_transformer import CausalTransformer, TransformerConfig
from dew_b200.nn.depth_residuals import DepthMix
from dew_b200.nn.dex import Dex, attach_dex, dex_parameters, head_entropies, set_progress

BASE = dict(vocab_size=40, emb_features=32, num_layers=2, num_heads=4, num_kv_heads=2, mlp_features=64, max_seq_len=32, qk_norm=False)


def _logits(m, t, **kw):
    y = m(t, **kw)
    return y[0] if isinstance(y, tuple) else y


def test_dex_starts_as_the_pretrained_function_and_anneals_in():
    torch.manual_seed(0)
    model = CausalTransformer(TransformerConfig(**BASE), dtype=torch.float32).train()
    tokens = torch.randint(0, 40, (2, 10))
    with torch.no_grad():
        before = _logits(model, tokens)
    made = attach_dex(model, {0: [1, 3], 1: [0]}, anneal_steps=10)
    assert len(made) == 2 and made[0].lambda_init == pytest.approx(0.8 - 0.6 * 2.718281828 ** 0.0, abs=1e-6)
    with torch.no_grad():
        assert torch.equal(_logits(model, tokens), before)               # step 0: lambda is 0
    set_progress(model, 5)
    d = made[0]
    assert float(d.strength()) == pytest.approx(0.5 * 0.5 * d.lambda_init + 0.5 * float(d.lambda_learn))
    with torch.no_grad():
        mid = _logits(model, tokens)
    assert not torch.allclose(mid, before)
    set_progress(model, 50)
    assert float(d.strength()) == pytest.approx(float(d.lambda_learn))
    model.eval()
    set_progress(model, 0)
    assert float(d.strength()) == pytest.approx(float(d.lambda_learn))   # outside training: the anneal's end
    # only the chosen heads change
    o = torch.randn(2, 5, 4, 8)
    out = d.train()(o)
    set_progress(model, 5)
    out = d(o)
    assert torch.equal(out[:, :, [0, 2]], o[:, :, [0, 2]]) and not torch.allclose(out[:, :, [1, 3]], o[:, :, [1, 3]])
    want = o[:, :, 1] - float(d.strength()) * (o[:, :, 1] @ d.weight[0])
    assert torch.allclose(out[:, :, 1], want, atol=1e-6)
    params = dex_parameters(model)
    assert any(p is d.weight for p in params) and any(p is model.layers[0].mixer.o_proj.weight for p in params)
    model.train()
    _logits(model, tokens).sum().backward()
    assert d.weight.grad.abs().sum() > 0 and d.lambda_learn.grad is not None
    with pytest.raises(TypeError, match="softmax attention"):
        hybrid = CausalTransformer(TransformerConfig(layer_types=("gla",), mixer_options=dict(num_heads=2), **BASE), dtype=torch.float32)
        attach_dex(hybrid, {0: [0]})


def test_head_entropies():
    q = torch.zeros(1, 6, 2, 4)
    k = torch.randn(1, 6, 1, 4)
    q[:, :, 1] = 50.0 * k[:, :, 0]                                        # head 1 attends sharply, head 0 uniformly
    e = head_entropies(q, k)
    uniform = torch.log(torch.arange(1, 7).float()).mean()
    assert float(e[0]) == pytest.approx(float(uniform), abs=1e-5) and float(e[1]) < float(e[0])


def test_depth_mix_averages_at_zero_kernel_and_selects_with_one():
    torch.manual_seed(0)
    mix = DepthMix(8)
    a, b, c = torch.randn(2, 3, 8), torch.randn(2, 3, 8), torch.randn(2, 3, 8)
    assert torch.allclose(mix([a, b, c]), (a + b + c) / 3, atol=1e-6)
    assert mix([a]) is a
    with torch.no_grad():
        mix.kernel.copy_(torch.randn(8))
    v = torch.stack([a, b, c], 2)
    k = v / (v.pow(2).mean(-1, keepdim=True) + 1e-6).sqrt()
    w = torch.softmax(k @ (mix.scale * mix.kernel), -1)
    assert torch.allclose(mix([a, b, c]), (w[..., None] * v).sum(2), atol=1e-6)


def test_decoder_with_block_attention_residuals():
    torch.manual_seed(0)
    cfg = TransformerConfig(**dict(BASE, num_layers=4), depth_residual_block=2)
    model = CausalTransformer(cfg, dtype=torch.float32)
    assert len(model.depth_sites.mixer) == 4
    tokens = torch.randint(0, 40, (2, 9))
    y = _logits(model, tokens)
    assert y.shape == (2, 9, 40)
    # by hand, layer by layer
    with torch.no_grad():
        h = model.embed(tokens)
        cos, sin = model.rope_tables(h.device)
        blocks, partial = [], h
        for i, layer in enumerate(model.layers):
            a = layer.mixer(layer.input_norm(model.depth_sites.mixer[i](blocks + [partial])), cos, sin, None, None, None, i)
            if i % 2 == 0:
                blocks.append(partial)
                partial = a
            else:
                partial = partial + a
            partial = partial + layer.mlp(layer.post_norm(model.depth_sites.mlp[i](blocks + [partial])))
        want = model.logits(model.final_norm(model.depth_sites.out(blocks + [partial])))
        assert len(blocks) == 2
    assert torch.allclose(y, want, atol=1e-5)
    y.logsumexp(-1).sum().backward()
    assert model.depth_sites.out.kernel.grad is not None and model.depth_sites.mixer[3].kernel.grad.abs().sum() > 0
    with pytest.raises(NotImplementedError, match="plain pre-norm"):
        CausalTransformer(TransformerConfig(**BASE, depth_residual_block=2, sandwich_norm=True))
