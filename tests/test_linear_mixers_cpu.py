"""GLA, DeltaNet and RWKV-7: chunked forms against their step-by-step recurrences, state carrying, and the mixers inside the decoder."""
import torch

from dew_b200.models import CausalTransformer
from dew_b200.nn.linear_mixers import DeltaNet, GatedLinearAttention, RWKV7, gla_chunked, gla_recurrent, rwkv7_recurrent
from dew_b200.ops import scan


def test_gla_chunked_matches_the_recurrence_and_carries_state():
    torch.manual_seed(0)
    B, T, H, dk, dv = 2, 70, 3, 8, 6
    q, k, v = torch.randn(B, T, H, dk), torch.randn(B, T, H, dk), torch.randn(B, T, H, dv)
    log_a = torch.nn.functional.logsigmoid(torch.randn(B, T, H, dk) * 2)
    o_ref, s_ref = gla_recurrent(q, k, v, log_a)
    o, s = gla_chunked(q, k, v, log_a, chunk=16)
    assert torch.allclose(o, o_ref, atol=1e-4, rtol=1e-4) and torch.allclose(s, s_ref, atol=1e-4, rtol=1e-4)
    # strong forgetting (gates near zero) stays finite: differences of cumulative gates are taken per pair, never exponentiated alone
    harsh = torch.full_like(log_a, -8.0)
    oh, _ = gla_chunked(q, k, v, harsh, chunk=32)
    assert torch.isfinite(oh).all() and torch.allclose(oh, gla_recurrent(q, k, v, harsh)[0], atol=1e-4)
    # two halves with the state carried equal the whole
    o1, s1 = gla_chunked(q[:, :40], k[:, :40], v[:, :40], log_a[:, :40], chunk=16)
    o2, s2 = gla_chunked(q[:, 40:], k[:, 40:], v[:, 40:], log_a[:, 40:], state=s1, chunk=16)
    assert torch.allclose(torch.cat([o1, o2], 1), o_ref, atol=1e-4) and torch.allclose(s2, s_ref, atol=1e-4)
    # gradients agree too
    qa, qb = q.clone().requires_grad_(), q.clone().requires_grad_()
    gla_chunked(qa, k, v, log_a, chunk=16)[0].pow(2).sum().backward()
    gla_recurrent(qb, k, v, log_a)[0].pow(2).sum().backward()
    assert torch.allclose(qa.grad, qb.grad, atol=1e-3, rtol=1e-3)


def test_gla_module_restarts_at_document_boundaries():
    torch.manual_seed(0)
    m = GatedLinearAttention(32, num_heads=2)
    a, b = torch.randn(1, 9, 32), torch.randn(1, 7, 32)
    packed = m(torch.cat([a, b], 1), segment_ids=torch.tensor([[1] * 9 + [2] * 7]))
    assert torch.allclose(packed[:, :9], m(a), atol=1e-5) and torch.allclose(packed[:, 9:], m(b), atol=1e-4)


def test_delta_rule_is_the_gated_rule_without_forgetting():
    torch.manual_seed(0)
    m = DeltaNet(32, num_heads=2, head_dim=16)
    x = torch.randn(2, 20, 32)
    out = m(x)
    assert out.shape == (2, 20, 32)
    # against the explicit recurrence S <- S (I - beta k k^T) + beta k^T v
    qkv = m.conv1d(m.qkv_proj(x), None, None)
    q, k, v = (t.reshape(2, 20, 2, 16) for t in qkv.chunk(3, -1))
    q, k = torch.nn.functional.normalize(q.float(), dim=-1), torch.nn.functional.normalize(k.float(), dim=-1)
    beta = torch.sigmoid(m.beta_proj(x).float())
    S = torch.zeros(2, 2, 16, 16)
    outs = []
    for t in range(20):
        kt, vt, bt = k[:, t], v[:, t].float(), beta[:, t][..., None]
        pred = torch.einsum("bhkv,bhk->bhv", S, kt)
        S = S + torch.einsum("bhk,bhv->bhkv", kt, bt * (vt - pred))
        outs.append(torch.einsum("bhkv,bhk->bhv", S, q[:, t]) * 16 ** -0.5)
    want = m.o_proj(m.norm(torch.stack(outs, 1)).reshape(2, 20, 32))
    assert torch.allclose(out, want, atol=1e-4, rtol=1e-3)


def test_rwkv7_recurrence_and_block():
    torch.manual_seed(0)
    B, T, H, d = 2, 6, 2, 4
    r, k, v = torch.randn(B, T, H, d), torch.randn(B, T, H, d), torch.randn(B, T, H, d)
    w, a = torch.rand(B, T, H, d) * 0.5 + 0.5, torch.rand(B, T, H, d)
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, d), dim=-1)
    o, S = rwkv7_recurrent(r, w, k, v, kk, a)
    # the state's update written out with matrices
    M = torch.zeros(B, H, d, d)
    for t in range(T):
        trans = torch.diag_embed(w[:, t]) - torch.einsum("bhk,bhj->bhkj", kk[:, t], a[:, t] * kk[:, t])
        M = M @ trans + torch.einsum("bhv,bhk->bhvk", v[:, t], k[:, t])
        assert torch.allclose(o[:, t], torch.einsum("bhvk,bhk->bhv", M, r[:, t]), atol=1e-5)
    assert torch.allclose(S, M, atol=1e-5)
    # with a = 0 (nothing removed) and w = 1 it is plain linear attention
    plain, _ = rwkv7_recurrent(r, torch.ones_like(w), k, v, kk, torch.zeros_like(a))
    cum = torch.einsum("bthv,bthk->bthvk", v, k).cumsum(1)
    assert torch.allclose(plain, torch.einsum("bthvk,bthk->bthv", cum, r), atol=1e-5)
    block = RWKV7(32, num_heads=2)
    x = torch.randn(2, 10, 32)
    y = block(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    later = x.clone(); later[:, 6:] = 0
    assert torch.allclose(block(later)[:, :6], y[:, :6], atol=1e-5)       # causal


def test_linear_mixers_as_decoder_layers():
    torch.manual_seed(0)
    tokens = torch.randint(0, 32, (2, 12))
    for kind in ("gla", "delta", "rwkv7"):
        m = CausalTransformer(vocab_size=32, emb_features=32, num_layers=2, num_heads=2, head_dim=16, mlp_features=64, max_seq_len=16,
                              layer_types=(kind, "attention"), qk_norm=False)
        logits = m(tokens)
        other = tokens.clone(); other[:, 8:] = (other[:, 8:] + 1) % 32
        assert logits.shape == (2, 12, 32) and torch.allclose(m(other)[:, :8], logits[:, :8], atol=1e-4), kind
        logits.float().pow(2).mean().backward()
        assert all(p.grad is not None for n, p in m.layers[0].mixer.named_parameters() if "v0" not in n and "v_lora" not in n), kind
