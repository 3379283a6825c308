"""Lightning attention, S5 and Mamba-3: parallel forms against their step-by-step recurrences."""
import torch

from dew_b200.nn import recurrent_mixers as R


def test_lightning_attention_matches_recurrence_and_slopes():
    torch.manual_seed(0)
    B, T, H, Dk, Dv = 2, 150, 4, 16, 8
    q, k = torch.randn(B, T, H, Dk, dtype=torch.float64), torch.randn(B, T, H, Dk, dtype=torch.float64)
    v = torch.randn(B, T, H, Dv, dtype=torch.float64)
    rate = R.alibi_slopes(H).double()
    s0 = torch.randn(B, H, Dk, Dv, dtype=torch.float64) * 0.1
    o1, s1 = R.lightning_recurrent(q, k, v, rate, s0)
    o2, s2 = R.lightning_attention(q, k, v, rate, s0)
    assert torch.allclose(o1, o2, atol=1e-9) and torch.allclose(s1, s2, atol=1e-9)
    assert torch.allclose(R.alibi_slopes(8), torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    assert R.alibi_slopes(6).shape == (6,)
    layer = R.LightningAttention(32, num_heads=4, head_dim=8, depth=1, layers=4)
    x = torch.randn(2, 20, 32, requires_grad=True)
    layer(x).pow(2).sum().backward()
    assert x.grad.abs().sum() > 0


def test_s5_scan_matches_recurrence():
    torch.manual_seed(1)
    layer = R.S5Layer(12, state_dim=16)
    u = torch.randn(2, 37, 12)
    assert torch.allclose(layer(u), layer(u, recurrent=True), atol=1e-4)
    a = torch.rand(2, 9, 3) * 0.9
    b = torch.randn(2, 9, 3)
    h, ref = torch.zeros(2, 3), []
    for t in range(9):
        h = a[:, t] * h + b[:, t]
        ref.append(h)
    assert torch.allclose(R.affine_scan(a, b, 1), torch.stack(ref, 1), atol=1e-6)


def test_mamba3_parallel_matches_complex_recurrence():
    torch.manual_seed(2)
    B, T, H, P, N = 2, 40, 3, 5, 8
    f = torch.float64
    x = torch.randn(B, T, H, P, dtype=f)
    dt = torch.nn.functional.softplus(torch.randn(B, T, H, dtype=f))
    A = -torch.rand(H, dtype=f) - 0.1
    Bm, Cm = torch.randn(B, T, H, N, dtype=f), torch.randn(B, T, H, N, dtype=f)
    theta = torch.randn(B, T, H, N // 2, dtype=f)
    lam = torch.rand(B, T, H, dtype=f)
    y1 = R.mamba3_recurrent(x, dt, A, Bm, Cm, theta, lam)
    y2 = R.mamba3_parallel(x, dt, A, Bm, Cm, theta, lam)
    assert torch.allclose(y1, y2, atol=1e-9), float((y1 - y2).abs().max())
    layer = R.Mamba3(16, state_dim=8, head_dim=8)
    xx = torch.randn(2, 12, 16)
    assert torch.allclose(layer(xx), layer(xx, recurrent=True), atol=1e-4)


def test_mla_latent_cache_decodes_like_the_full_forward():
    """Multi-head latent attention with a latent KV cache: prefill a prompt, then decode token by token through the absorbed
    form (queries folded through the key up-projection, values rebuilt after the sum); every step equals the row of the full
    causal forward, and the cache holds kv_latent + rope_dim numbers per token (src/dew/nn/mla.py)."""
    import torch
    from dew_b200 import ops
    from dew_b200.nn.kv_cache import KVCache, KVStore
    from dew_b200.nn.mla import MultiHeadLatentAttention
    torch.manual_seed(0)
    m = MultiHeadLatentAttention(32, 4, kv_latent=16, q_latent=24, nope_dim=8, rope_dim=4, v_dim=8)
    cos, sin = ops.rope_tables(32, 4, 10000.0, torch.device("cpu"))
    x = torch.randn(2, 12, 32)
    pos = torch.arange(12)[None].expand(2, 12)
    full = m(x, cos, sin, pos)
    store = KVStore(KVCache(), 1, 2, 32, 1, 4, torch.float32, "cpu")
    first = m(x[:, :7], cos, sin, pos[:, :7], cache=store, layer=0)
    assert torch.allclose(first, full[:, :7], atol=1e-5)
    for t in range(7, 12):
        step = m(x[:, t:t + 1], cos, sin, pos[:, t:t + 1], cache=store, layer=0)
        assert torch.allclose(step[:, 0], full[:, t], atol=1e-5), t
    assert store.latent(0, 20).shape == (2, 32, 20)            # 16 latent + 4 rotary numbers per token, no per-head keys / values
