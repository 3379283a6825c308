"""Cross-pass messages: a looped decoder whose later passes read the block summaries the pass before left."""
import torch

from dew_b200.models.causal_transformer import CausalTransformer, Loop, TransformerConfig
from dew_b200.nn.cross_pass import CrossPassMerge

BASE = dict(vocab_size=40, emb_features=32, num_layers=4, num_heads=4, mlp_features=64, max_seq_len=32, qk_norm=False)


def _logits(m, t, **kw):
    y = m(t, **kw)
    return y[0] if isinstance(y, tuple) else y


def test_merge_starts_as_the_identity_and_follows_its_formula():
    torch.manual_seed(0)
    merge = CrossPassMerge(16, rank=4)
    u, bank = torch.randn(2, 5, 16) * 3, torch.randn(2, 5, 3, 16)
    assert torch.allclose(merge(u, bank), u, atol=1e-6)
    with torch.no_grad():
        merge.w_out.normal_(0, 0.3)
        merge.query.normal_(0, 1.0)
    k = bank / (bank.pow(2).mean(-1, keepdim=True) + 1e-6).sqrt()
    m = (torch.softmax(k @ merge.query, -1)[..., None] * bank).sum(-2)
    m = m / (m.pow(2).mean(-1, keepdim=True) + 1e-6).sqrt()
    sigma = (u.pow(2).mean(-1, keepdim=True) + 1e-6).sqrt()
    h = (u / sigma) @ merge.w_u + m @ merge.w_m
    f, g, a = torch.tanh(h @ merge.w_out).chunk(3, -1)
    assert torch.allclose(merge(u, bank), (1 - f) * u + sigma * (g * m + a), atol=1e-5)
    assert abs(float(merge.message(bank).pow(2).mean(-1).sqrt().mean()) - 1.0) < 1e-3


def test_looped_decoder_with_messages():
    torch.manual_seed(0)
    plain = CausalTransformer(TransformerConfig(**BASE), dtype=torch.float32).eval()
    cfg = TransformerConfig(**BASE, loop=Loop(steps=3, first=1, end=3, messages=1, message_rank=4))
    model = CausalTransformer(cfg, dtype=torch.float32).eval()
    assert model.layers[0].cross is None and len(model.layers[1].cross) == 2 and model.layers[3].cross is None
    model.load_state_dict(plain.state_dict(), strict=False)
    tokens = torch.randint(0, 40, (2, 9))
    with torch.no_grad():
        # gates at zero: every pass starts from the prelude and is the first pass again - the unlooped decoder's own function
        assert torch.allclose(_logits(model, tokens), _logits(plain, tokens), atol=1e-5)
        per_pass = model(tokens, passes=True)
        assert len(per_pass) == 3 and torch.allclose(per_pass[0], per_pass[2], atol=1e-6)
        for layer in model.layers[1:3]:
            for merge in layer.cross:
                merge.w_out.normal_(0, 0.2)
        per_pass = model(tokens, passes=True)
        assert torch.allclose(per_pass[0], _logits(plain, tokens), atol=1e-5)          # the first pass reads no bank
        assert not torch.allclose(per_pass[1], per_pass[0], atol=1e-4) and not torch.allclose(per_pass[2], per_pass[1], atol=1e-5)
    model.train()
    _logits(model, tokens).logsumexp(-1).sum().backward()
    assert model.layers[1].cross[0].w_out.grad.abs().sum() > 0 and model.layers[2].cross[1].query.grad is not None
    # remat recomputes each pass with the bank that pass read
    torch.manual_seed(0)
    rm = CausalTransformer(TransformerConfig(**BASE, remat=True, loop=Loop(steps=3, first=1, end=3, messages=1, message_rank=4)), dtype=torch.float32)
    rm.load_state_dict(model.state_dict())
    model.zero_grad()
    _logits(model, tokens, train=True).logsumexp(-1).sum().backward()
    _logits(rm, tokens, train=True).logsumexp(-1).sum().backward()
    for (n, a), (_, b) in zip(model.named_parameters(), rm.named_parameters()):
        if a.grad is not None:
            assert torch.allclose(a.grad, b.grad, atol=1e-5), n
