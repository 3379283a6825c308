"""The transformer state-space model: the window form and the stepped form are one function; episodes do not see each other; the prior sees no observation."""
import torch

from dew_b200.objectives.rl.tssm import TSSM


def _model():
    torch.manual_seed(0)
    m = TSSM(embed=12, action=3, deter=32, stoch=4, classes=6, layers=2, heads=4, hidden=32).eval()
    with torch.no_grad():
        m.start.normal_(0, 0.5)
    return m


def test_window_and_stepped_forms_agree_and_episodes_are_isolated():
    m = _model()
    N, T = 2, 9
    embed, actions = torch.randn(N, T, 12), torch.randn(N, T, 3)
    first = torch.zeros(N, T, dtype=torch.bool)
    first[0, 4] = True
    first[1, 6] = True
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        h, z, prior, post = m.observe(embed, actions, first, g)
        assert h.shape == (N, T, 32) and z.shape == (N, T, 24) and prior.shape == post.shape == (N, T, 4, 6)
        cache = m.initial(N, "cpu")
        hs = []
        for t in range(T):
            z_prev = z[:, t - 1] if t else torch.zeros(N, 24)
            a_prev = actions[:, t - 1] if t else torch.zeros(N, 3)
            ht, pr, cache = m.step(cache, z_prev, a_prev, first[:, t])
            hs.append(ht)
            assert torch.allclose(pr, prior[:, t], atol=1e-5)
        assert torch.allclose(torch.stack(hs, 1), h, atol=1e-5)
        # what happened before an episode's start does not reach it
        other_e, other_a = embed.clone(), actions.clone()
        other_e[0, :4], other_a[0, :4] = torch.randn(4, 12), torch.randn(4, 3)
        g2 = torch.Generator().manual_seed(5)
        h2, z2, _, _ = m.observe(other_e, other_a, first, g2)
        assert torch.allclose(h2[0, 4], h[0, 4]) and not torch.allclose(h2[0, 3], h[0, 3])
        # the deterministic state holds nothing of its own step's observation
        shifted = embed.clone()
        shifted[:, 5] += 1.0
        g3 = torch.Generator().manual_seed(5)
        h3, _, _, _ = m.observe(shifted, actions, first, g3)
        assert torch.allclose(h3[:, :6], h[:, :6], atol=1e-6)
        trimmed = cache.trimmed(3)
        assert trimmed.k[0].shape[1] == 3 and trimmed.episode.shape == (N, 3)


def test_imagination_and_gradients():
    m = _model().train()
    N = 3
    embed, actions = torch.randn(N, 5, 12), torch.randn(N, 5, 3)
    first = torch.zeros(N, 5, dtype=torch.bool)
    h, z, prior, post = m.observe(embed, actions, first)
    kl = (post.exp() * (post - prior.detach())).sum((-1, -2)).mean() + (post.detach().exp() * (post.detach() - prior)).sum((-1, -2)).mean()
    kl.backward()
    assert m.blocks[0].qkv.weight.grad.abs().sum() > 0 and m.post[0].weight.grad.abs().sum() > 0 and m.start.grad is not None
    with torch.no_grad():
        cache = m.initial(N, "cpu")
        for t in range(5):
            _, _, cache = m.step(cache, z[:, t - 1] if t else torch.zeros(N, 24), actions[:, t - 1] if t else torch.zeros(N, 3), first[:, t])
        feats, acts = m.imagine(cache, z[:, -1], lambda h, zz: torch.tanh(zz[:, :3]), steps=4)
    assert feats.shape == (4, N, m.features) and acts.shape == (4, N, 3) and torch.isfinite(feats).all()
