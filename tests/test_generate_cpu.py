"""Text generation: cached decoding equals recomputing from scratch; transforms; strategies."""
import torch

import dew_b200 as dew
from dew_b200.models import CausalTransformer
from dew_b200.nn.kv_cache import KVCache
from dew_b200.sampling.text import Beam, Sampling, Speculative, generate, transform_logits


def _model(seed=0, layers=2):
    torch.manual_seed(seed)
    return CausalTransformer(vocab_size=97, emb_features=32, num_layers=layers, num_heads=4, num_kv_heads=2, mlp_features=64,
                             max_seq_len=64, tie_embeddings=True).eval()


def _greedy_no_cache(model, prompt, n):
    seq = list(prompt)
    with torch.no_grad():
        for _ in range(n):
            seq.append(int(model(torch.tensor([seq]))[0, -1].argmax()))
    return seq


def test_greedy_generation_with_paged_cache_matches_recompute():
    m = _model()
    prompts = [[5, 9, 3], [7, 1, 2, 8, 4, 6], [11]]
    for spec in (None, KVCache(page_size=4)):
        g = generate(m, None, prompts, 8, sampling=Sampling(temperature=0.0), kv_cache=spec)
        for r, p in enumerate(prompts):
            assert g.tokens[r, : int(g.lengths[r])].tolist() == _greedy_no_cache(m, p, 8)


def test_sampling_is_keyed_per_row_and_reproducible():
    m = _model(1)
    s = Sampling(temperature=0.9, top_k=20, top_p=0.95)
    a = generate(m, None, [[1, 2, 3], [4, 5]], 6, key=7, sampling=s)
    b = generate(m, None, [[1, 2, 3], [4, 5]], 6, key=7, sampling=s)
    assert torch.equal(a.tokens, b.tokens)
    alone = generate(m, None, [[1, 2, 3]], 6, key=7, sampling=s)
    assert alone.tokens[0, :9].tolist() == a.tokens[0, :9].tolist()     # row 0 does not depend on its batch mates


def test_eos_stops_and_transforms_mask():
    m = _model(2)
    first = _greedy_no_cache(m, [3, 4], 1)[-1]
    g = generate(m, None, [[3, 4]], 5, sampling=Sampling(temperature=0.0, eos_token_ids=[first]))
    assert bool(g.terminated[0]) and int(g.lengths[0]) == 3
    logits = -torch.arange(10.0)[None] * 0.1; logits[0, 3] = 5.0
    hist, hl = torch.tensor([[3, 3, 0]]), torch.tensor([2])
    x = transform_logits(logits, hist, hl, Sampling(temperature=1.0, repetition_penalty=2.0, top_k=3), 0)
    assert x[0, 3] == 2.5 and torch.isinf(x[0]).sum() == 7
    y = transform_logits(logits, hist, hl, Sampling(temperature=1.0, no_repeat_ngram_size=2), 0)
    assert torch.isinf(y[0, 3])                                         # "3 3" already occurred after a 3


def test_beam_and_speculative():
    m, d = _model(3), _model(4, layers=1)
    g = Beam(beams=3).run(m, None, [[2, 3, 4]], 5)
    assert int(g.lengths[0]) == 8
    sp = Speculative(draft=d, lookahead=3).run(m, None, [[2, 3, 4]], 6)
    assert sp.tokens[0, :9].tolist() == _greedy_no_cache(m, [2, 3, 4], 6)    # exact for greedy decoding


def test_sample_rows_reference_path_matches_transform_logits():
    """The sampling op's CPU path keeps the same tokens as the Sampling transforms (no ties in random logits)."""
    import torch
    from dew_b200.ops import sample as S
    from dew_b200.sampling.text import Sampling, transform_logits
    torch.manual_seed(0)
    logits = torch.randn(5, 300) * 2
    s = Sampling(temperature=0.8, top_k=40, top_p=0.9, min_p=0.01)
    a = S.filtered_reference(logits, s.temperature, s.top_k, s.top_p, s.min_p)
    b = transform_logits(logits, torch.zeros(5, 1, dtype=torch.long), torch.zeros(5, dtype=torch.long), s, 0)
    assert torch.equal(torch.isfinite(a), torch.isfinite(b))
    tok = S.sample_rows(logits, torch.rand(5), s.temperature, s.top_k, s.top_p, s.min_p)
    assert torch.isfinite(a.gather(-1, tok[:, None])).all()


def _tiny_lm(seed):
    import torch
    from dew_b200.models import CausalTransformer
    torch.manual_seed(seed)
    return CausalTransformer(vocab_size=40, emb_features=32, num_layers=2, num_heads=4, head_dim=8, mlp_features=64, max_seq_len=64).eval()


def test_tree_speculative_equals_greedy_and_mask_shape():
    import torch
    from dew_b200.sampling.text import Sampling, TreeSpeculative, generate
    target, draft = _tiny_lm(0), _tiny_lm(1)
    prompts = [[1, 2, 3, 4], [5, 6, 7]]
    want = generate(target, None, prompts, 10, sampling=Sampling(temperature=0.0))
    got = TreeSpeculative(draft=draft, branching=2, depth=2).run(target, None, prompts, 10, sampling=Sampling(temperature=0.0))
    for r in range(2):
        assert got.new_tokens(r).tolist() == want.new_tokens(r).tolist()
    same = TreeSpeculative(draft=target, branching=2, depth=3).run(target, None, prompts, 9, sampling=Sampling(temperature=0.0))
    assert same.accepted_per_round == 3.0                      # the target as its own draft: every level is accepted
    m = TreeSpeculative.tree_mask(3, [-1, -1, 0, 0, 1, 1])
    assert m.shape == (9, 9) and bool(m[3 + 4, 3 + 1]) and not bool(m[3 + 4, 3 + 0]) and bool(m[3 + 2, 3 + 0])


def test_grammar_guided_decoding_stays_inside_the_language():
    import torch
    from dew_b200.sampling.guided import Grammar, guided_generate
    vocab = ["", "yes", "no", "ma", "ybe", "!", " ", "x"] + [f"t{i}" for i in range(32)]
    g = Grammar.from_regex(r"(yes|no|maybe)!", vocab)
    model = _tiny_lm(3)
    for seed in range(4):
        gen = torch.Generator().manual_seed(seed)
        toks, ok = guided_generate(model, [1, 2], g, 6, eos_token_id=None, temperature=1.0, generator=gen)
        text = "".join(vocab[t] for t in toks)
        assert ok and text in ("yes!", "no!", "maybe!")
    t = Grammar.from_transitions({0: {5: 1}, 1: {6: 1, 7: 2}, 2: {}}, 0, {2}, 40)
    assert t.mask(1).nonzero().flatten().tolist() == [6, 7] and t.advance(1, 7) == 2 and t.accepting(2) and t.dead(2)
