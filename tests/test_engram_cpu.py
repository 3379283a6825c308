"""Engram: exact n-gram hashing, look-back that stops at boundaries, a causal gated write, and a decoder that learns a bigram rule with it."""
import torch

from dew_b200.models.causal_transformer import CausalTransformer, TransformerConfig
from dew_b200.nn.engram import Engram, compressed_token_map, lookback, ngram_buckets, odd_multipliers, primes_below, splitmix64


def test_hashes_are_exact_integer_arithmetic():
    assert splitmix64(0, 2) == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4]          # the published first outputs of SplitMix64 from seed 0
    mult = odd_multipliers(7, 3, 4)
    assert all(m % 2 == 1 and m < 1 << 31 for m in mult) and mult != odd_multipliers(7, 4, 4)
    primes = primes_below(1000, 6)
    assert primes == [997, 991, 983, 977, 971, 967]
    torch.manual_seed(0)
    tokens = torch.randint(0, (1 << 24) - 1, (2, 9))
    window = lookback(tokens, 4, pad_id=0)
    got = ngram_buckets(window, mult, torch.tensor(primes).view(3, 2))
    for b in range(2):
        for t in range(9):
            ids = [int(tokens[b, t - k]) if t - k >= 0 else 0 for k in range(4)]
            run = ids[0] * mult[0]
            for n in range(1, 4):
                run ^= ids[n] * mult[n]
                for head in range(2):
                    assert int(got[b, t, n - 1, head]) == run % primes[(n - 1) * 2 + head]


def test_lookback_stops_at_starts_boundaries_and_stop_tokens():
    tokens = torch.tensor([[5, 6, 7, 8, 9, 10]])
    seg = torch.tensor([[0, 0, 0, 1, 1, 1]])
    w = lookback(tokens, 3, pad_id=99, segment_ids=seg)
    assert w[0, 0].tolist() == [5, 99, 99] and w[0, 2].tolist() == [7, 6, 5]
    assert w[0, 3].tolist() == [8, 99, 99] and w[0, 4].tolist() == [9, 8, 99]
    w = lookback(tokens, 4, pad_id=99, stop_id=7)
    assert w[0, 3].tolist() == [8, 99, 99, 99]                 # behind the stop token nothing is read, even further back
    assert w[0, 5].tolist() == [10, 9, 8, 99]
    m = compressed_token_map(["Hello", " hello", "▁HELLO", "world", "Ｗorld"])
    assert m.tolist() == [0, 0, 0, 1, 1]


def test_write_is_causal_gated_and_trainable():
    torch.manual_seed(0)
    e = Engram(32, 100, layer=2, max_ngram=3, heads=2, buckets=257, width=8, conv=3)
    h = torch.randn(2, 10, 32)
    tokens = torch.randint(0, 100, (2, 10))
    assert torch.equal(e(h, tokens), h)                         # value projection starts at zero: the layer starts as the identity
    with torch.no_grad():
        e.value.weight.normal_(0, 0.2)
        e.conv.weight.normal_(0, 0.2)
    out = e(h, tokens)
    other = tokens.clone()
    other[:, 6:] = torch.randint(0, 100, (2, 4))
    assert torch.equal(e(h, other)[:, :6], out[:, :6]) and not torch.equal(e(h, other)[:, 6:], out[:, 6:])
    rows = e.rows(tokens)
    assert rows.shape == (2, 10, 2, 2) and int(rows.max()) < e.table.num_embeddings
    assert torch.equal(rows[0, 5], e.rows(tokens[:1, 3:6])[0, 2])           # a trigram's rows depend on its three tokens alone
    out.sum().backward()
    assert e.table.weight.grad.abs().sum() > 0 and e.key.weight.grad.abs().sum() > 0


def test_decoder_with_engram_learns_a_bigram_rule():
    """Next token = (previous + current) mod V: a function of the bigram, which one shallow layer without attention to rely on learns from the
    n-gram memory."""
    torch.manual_seed(0)
    V = 23
    cfg = TransformerConfig(vocab_size=V, emb_features=32, num_layers=1, num_heads=2, mlp_features=64, max_seq_len=32, qk_norm=False,
                            engram=dict(layers=[0], max_ngram=2, heads=2, buckets=1031, width=16))
    model = CausalTransformer(cfg, dtype=torch.float32)
    assert set(model.engrams) == {"0"}
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)

    def batch(n):
        x = torch.randint(0, V, (n, 2))
        seq = [x[:, 0], x[:, 1]]
        for _ in range(14):
            seq.append((seq[-1] + seq[-2]) % V)
        return torch.stack(seq, 1)
    for _ in range(300):
        t = batch(32)
        y = model(t[:, :-1])
        y = y[0] if isinstance(y, tuple) else y
        loss = torch.nn.functional.cross_entropy(y[:, 1:].reshape(-1, V), t[:, 2:].reshape(-1))
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(loss) < 0.3, float(loss)
    import pytest
    with pytest.raises(NotImplementedError, match="whole sequences"):
        model.hidden(None, embeddings=torch.randn(1, 4, 32))
