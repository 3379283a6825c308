"""The in-context memory layer: analytic inner gradients against autograd, the chunk form against the token-by-token definition,
document resets, streaming state, and the delta-rule property of the linear l2 memory."""
import pytest
import torch

from dew_b200.models.causal_transformer import CausalTransformer, TransformerConfig
from dew_b200.nn.memory import NeuralMemory, inner_forward, inner_gradients


@pytest.mark.parametrize("hidden", [0, 12])
@pytest.mark.parametrize("objective", ["l2", "dot"])
def test_inner_gradients_match_autograd(hidden, objective):
    torch.manual_seed(0)
    shapes = [(8, 8)] if hidden == 0 else [(8, hidden), (hidden, 8)]
    W = [torch.randn(3, 2, *s, dtype=torch.float64, requires_grad=True) for s in shapes]
    k, v = torch.randn(3, 2, 8, dtype=torch.float64), torch.randn(3, 2, 8, dtype=torch.float64)
    p = inner_forward(W, k)
    loss = (0.5 * (p - v).pow(2).sum() if objective == "l2" else -(p * v).sum())
    want = torch.autograd.grad(loss, W)
    got = inner_gradients([w.detach() for w in W], k, v, objective)
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=1e-10)


@pytest.mark.parametrize("fields", [dict(), dict(hidden=10), dict(momentum=False), dict(retention=False), dict(commit=True), dict(objective="dot", hidden=6),
                                    dict(momentum=False, retention=False)])
def test_chunk_form_is_the_stepped_definition(fields):
    torch.manual_seed(0)
    m = NeuralMemory(32, num_heads=2, head_dim=8, chunk=5, **fields).double()
    with torch.no_grad():
        m.gate_proj.weight.normal_(0, 0.5)
        for p in m.initial:
            p.data = p.data.double().normal_(0, 0.3)
    x = torch.randn(2, 13, 32, dtype=torch.float64)
    views = [t.double() if t is not None else None for t in m.views(x)]
    a, sa = m.chunked(*views)
    b, sb = m.stepped(*views)
    assert torch.allclose(a, b, atol=1e-9), float((a - b).abs().max())
    for wa, wb in zip(sa["W"] + sa["S"], sb["W"] + sb["S"]):
        assert torch.allclose(wa, wb, atol=1e-9)
    assert sa["count"].tolist() == [13, 13]
    # gradients reach the outer parameters through the inner steps
    a.sum().backward()
    assert m.qkv_proj.weight.grad.abs().sum() > 0 and m.gate_proj.weight.grad.abs().sum() > 0 and m.initial[0].grad.abs().sum() > 0


def test_documents_reset_and_streams_carry_state():
    torch.manual_seed(0)
    m = NeuralMemory(32, num_heads=2, head_dim=8, chunk=4, hidden=6).eval()
    x = torch.randn(1, 14, 32)
    seg = torch.tensor([[0] * 6 + [1] * 8])
    with torch.no_grad():
        packed = m(x, segment_ids=seg)
        alone = m(x[:, 6:])
        assert torch.allclose(packed[:, 6:], alone, atol=1e-5)            # the second document reads a memory that never saw the first
        whole = m(x)
        first, state = m(x[:, :8], return_state=True)
        rest = []
        for t in range(8, 14):                                         # one token at a time from the carried state
            y, state = m(x[:, t:t + 1], state=state, return_state=True)
            rest.append(y)
        assert torch.allclose(torch.cat([first] + rest, 1), whole, atol=1e-5)
        part, state = m(x[:, :6], return_state=True)                   # stopping inside a chunk carries on through the stepped form
        tail, _ = m(x[:, 6:], state=state, return_state=True)
        assert torch.allclose(torch.cat([part, tail], 1), whole, atol=1e-5)


def test_linear_l2_memory_stores_what_it_is_shown():
    """One full step on a unit key makes the linear memory return the value for that key (the delta rule), and leaves an orthogonal key's reading alone."""
    torch.manual_seed(0)
    m = NeuralMemory(16, num_heads=1, head_dim=4, chunk=1, momentum=False, retention=False)
    k = torch.tensor([[[[1.0, 0, 0, 0]], [[0, 1.0, 0, 0]]]])            # [B=1, T=2, H=1, d]
    v = torch.tensor([[[[0.3, -1.0, 2.0, 0.5]], [[1.0, 1.0, -1.0, 0.0]]]])
    q = k.clone()
    theta = torch.ones(1, 2, 1)
    y, state = m.stepped(q, k, v, theta, None, None)
    assert torch.allclose(y, v, atol=1e-6)
    read_first = inner_forward(state["W"], k[:, 0])
    assert torch.allclose(read_first, v[:, 0], atol=1e-6)               # the second write did not disturb the first


def test_memory_as_a_decoder_layer():
    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=40, emb_features=32, num_layers=2, num_heads=2, mlp_features=64, max_seq_len=32, qk_norm=False,
                            layer_types=("memory", "attention"), mixer_options=dict(num_heads=2, head_dim=8, chunk=4, hidden=8))
    model = CausalTransformer(cfg, dtype=torch.float32)
    tokens = torch.randint(0, 40, (2, 12))
    y = model(tokens)
    y = y[0] if isinstance(y, tuple) else y
    assert y.shape == (2, 12, 40)
    y.logsumexp(-1).sum().backward()
    assert model.layers[0].mixer.initial[0].grad is not None
    other = tokens.clone()
    other[:, 8:] = (other[:, 8:] + 1) % 40
    with torch.no_grad():
        z = model(other)
    z = z[0] if isinstance(z, tuple) else z
    assert torch.allclose(z[:, :8], y[:, :8].detach(), atol=1e-5)        # causal
