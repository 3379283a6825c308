"""Rows that share a prefix are laid out with the prefix once: every row's outputs and the gradients equal the rows laid out whole."""
import pytest
import torch

from dew_b200.data.forked_rows import ForkedRows, Forks, group_by_prefix
from dew_b200.models.causal_transformer import CausalTransformer, TransformerConfig


def _logits(m, *a, **kw):
    y = m(*a, **kw)
    return y[0] if isinstance(y, tuple) else y


def test_grouping_and_layout():
    prompt_a, prompt_b = [5, 6, 7, 8, 9], [5, 6, 1, 2]
    rows = [prompt_a + [10, 11], prompt_b + [12], prompt_a + [13], prompt_a + [10, 14, 15], prompt_b + [16, 17], [30, 31]]
    groups = group_by_prefix(rows, min_prefix=3)
    assert sorted((p, sorted(ms)) for p, ms in groups) == [(0, [5]), (4, [1, 4]), (5, [0, 2, 3])]
    packed = ForkedRows.pack(rows, window=16, min_prefix=3)
    assert packed.whole == sum(len(r) for r in rows) and packed.laid == packed.whole - 2 * 5 - 4
    assert packed.saved == pytest.approx(14 / packed.whole)
    for i, r in enumerate(rows):                                   # every row's tokens and positions sit at its slots, in its order
        assert packed.tokens.reshape(-1)[packed.slots[i]].tolist() == r
        assert packed.positions.reshape(-1)[packed.slots[i]].tolist() == list(range(len(r)))
    vis = packed.forks.visible()
    flat_seg = packed.forks.segment_ids
    for i, r in enumerate(rows):                                   # a row's last token sees exactly the row
        w, last = int(packed.slots[i][-1]) // 16, int(packed.slots[i][-1]) % 16
        seen = vis[w, last].nonzero().reshape(-1) + w * 16
        assert sorted(seen.tolist()) == sorted(packed.slots[i].tolist())
    whole = ForkedRows.pack(rows, window=16, share=False)
    assert whole.laid == whole.whole and int((whole.forks.parent_ids >= 0).sum()) == 0
    with pytest.raises(ValueError, match="a window"):
        ForkedRows.pack([[1] * 20], window=16)
    # a row that is another's prefix keeps a token of its own
    p = ForkedRows.pack([[1, 2, 3], [1, 2, 3, 4, 5]], window=8)
    assert p.laid == 6 and p.tokens.reshape(-1)[p.slots[0]].tolist() == [1, 2, 3]


def test_model_outputs_and_gradients_equal_the_rows_laid_whole():
    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=50, emb_features=32, num_layers=2, num_heads=4, num_kv_heads=2, mlp_features=64, max_seq_len=64, qk_norm=True)
    model = CausalTransformer(cfg, dtype=torch.float32)
    prompt = torch.randint(0, 50, (9,)).tolist()
    other = torch.randint(0, 50, (6,)).tolist()
    rows = [prompt + torch.randint(0, 50, (n,)).tolist() for n in (4, 7, 2, 5)] + [other + torch.randint(0, 50, (n,)).tolist() for n in (3, 3)]
    packed = ForkedRows.pack(rows, window=40, min_prefix=4)
    assert packed.saved > 0.35 and packed.tokens.shape[0] == 1

    def loss_of(parts):
        return sum((p.logsumexp(-1) * torch.linspace(0.5, 1.5, p.shape[0])).sum() for p in parts)
    out = _logits(model, packed.tokens, positions=packed.positions, segment_ids=packed.forks)
    shared = packed.gathered(out)
    alone = [_logits(model, torch.tensor([r]))[0] for r in rows]
    for a, b in zip(shared, alone):
        assert torch.allclose(a, b, atol=2e-5), float((a - b).abs().max())
    g_shared = torch.autograd.grad(loss_of(shared), list(model.parameters()), allow_unused=True)
    g_alone = torch.autograd.grad(loss_of(alone), list(model.parameters()), allow_unused=True)
    for a, b in zip(g_shared, g_alone):
        if a is not None:
            assert torch.allclose(a, b, atol=2e-4 * max(1.0, float(b.abs().max()))), float((a - b).abs().max())
    padded, mask = packed.padded(out)
    assert padded.shape[:2] == (6, 16) and mask.sum(1).tolist() == [len(r) for r in rows]
    # a recurrent mixer cannot read forks
    hybrid = CausalTransformer(TransformerConfig(vocab_size=50, emb_features=32, num_layers=1, num_heads=4, mlp_features=64, max_seq_len=64, qk_norm=False,
                                                 layer_types=("gla",), mixer_options=dict(num_heads=2)), dtype=torch.float32)
    with pytest.raises(Exception):
        hybrid(packed.tokens, positions=packed.positions, segment_ids=packed.forks)


def test_grpo_with_a_shared_prompt_gives_the_same_loss_and_gradients():
    from dew_b200.objectives.base import Step
    from dew_b200.objectives.rl.policy import GRPO
    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=50, emb_features=32, num_layers=2, num_heads=4, mlp_features=64, max_seq_len=64, qk_norm=False)
    model = CausalTransformer(cfg, dtype=torch.float32)
    G, P, S = 4, 10, 18
    prompts = torch.randint(1, 50, (2, P))
    tokens = torch.zeros(2 * G, S, dtype=torch.long)
    mask = torch.zeros(2 * G, S)
    for i in range(2 * G):
        n = int(torch.randint(3, S - P + 1, ()))
        tokens[i, :P] = prompts[i // G]
        tokens[i, P:P + n] = torch.randint(1, 50, (n,))
        mask[i, P:P + n] = 1
    batch = dict(tokens=tokens, mask=mask, rewards=torch.randn(2 * G), old_logprobs=torch.randn(2 * G, S - 1) * 0.1 - 3.5)
    step = Step(step=0)
    results = []
    for share in (False, True):
        obj = GRPO(model, group=G, kl=0.0, share_prefix=share, min_prefix=4)
        stats, _ = obj.loss(None, batch, step)
        value = stats.total / stats.mass
        grads = torch.autograd.grad(value, list(model.parameters()), allow_unused=True)
        results.append((value.detach(), grads))
    assert torch.allclose(results[0][0], results[1][0], atol=1e-5)
    for a, b in zip(results[0][1], results[1][1]):
        if a is not None:
            assert torch.allclose(a, b, atol=1e-5 + 1e-4 * float(a.abs().max()))


def test_dpo_with_a_shared_prompt_gives_the_same_loss_and_gradients():
    from dew_b200.objectives.base import Step
    from dew_b200.objectives.rl.preference import DPO
    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=50, emb_features=32, num_layers=2, num_heads=4, mlp_features=64, max_seq_len=64, qk_norm=False)
    model = CausalTransformer(cfg, dtype=torch.float32)
    reference = {k: v.detach().clone() + 0.01 * torch.randn_like(v) for k, v in model.named_parameters()}
    B, P, S = 3, 9, 16
    chosen, rejected = torch.zeros(B, S, dtype=torch.long), torch.zeros(B, S, dtype=torch.long)
    cm, rm = torch.zeros(B, S), torch.zeros(B, S)
    for i in range(B):
        prompt = torch.randint(1, 50, (P,))
        nc, nr = int(torch.randint(2, S - P + 1, ())), int(torch.randint(2, S - P + 1, ()))
        chosen[i, :P], rejected[i, :P] = prompt, prompt
        chosen[i, P:P + nc], rejected[i, P:P + nr] = torch.randint(1, 50, (nc,)), torch.randint(1, 50, (nr,))
        cm[i, P:P + nc], rm[i, P:P + nr] = 1, 1
    batch = dict(chosen=chosen, rejected=rejected, chosen_mask=cm, rejected_mask=rm)
    from dew_b200.utils.trees import unflatten
    results = []
    for share in (False, True):
        obj = DPO(model, beta=0.5, share_prefix=share, min_prefix=4)
        stats, aux = obj.loss(None, batch, Step(step=0))
        value = stats.total / stats.mass
        results.append((value.detach(), torch.autograd.grad(value, list(model.parameters()), allow_unused=True)))
    assert torch.allclose(results[0][0], results[1][0], atol=1e-5)
    for a, b in zip(results[0][1], results[1][1]):
        if a is not None:
            assert torch.allclose(a, b, atol=1e-5 + 1e-4 * float(a.abs().max()))
