"""Entropy-bounded block generation for a block diffusion language model."""
import torch

from dew_b200.objectives.discrete import BlockDiffusionLM, entropy_bounded_choice


def test_entropy_bounded_choice():
    e = torch.tensor([[0.05, 0.9, 0.1, 0.2, 0.0], [0.5, 0.6, 0.7, 0.8, 0.9]])
    masked = torch.tensor([[True, True, True, True, False], [True, True, True, True, True]])
    chosen = entropy_bounded_choice(e, masked, 0.2)
    # row 0: rising 0.05, 0.1, 0.2, 0.9 -> sums less the largest 0, 0.05, 0.15, 0.35: three places; the unmasked place never
    assert chosen[0].tolist() == [True, False, True, True, False]
    assert chosen[1].tolist() == [True, False, False, False, False]        # all uncertain: only the most certain one
    assert entropy_bounded_choice(e, masked, 0.0).sum(-1).tolist() == [1, 1]
    assert entropy_bounded_choice(e, masked, 100.0).tolist() == masked.tolist()
    none = torch.zeros(1, 5, dtype=torch.bool)
    assert not bool(entropy_bounded_choice(e[:1], none, 1.0).any())


class Oracle(torch.nn.Module):
    """Predicts ``target`` at every place, sharply where ``sharp`` says and vaguely elsewhere - more sharply once the place before is known."""

    def __init__(self, target, sharp, vocab=12, mask_id=11):
        super().__init__()
        self.target, self.sharp, self.vocab, self.mask_id = target, sharp, vocab, mask_id

    def forward(self, tokens):
        R, L = tokens.shape
        logits = torch.zeros(R, L, self.vocab)
        for i in range(L):
            known_before = i == 0 or bool((tokens[:, i - 1] != self.mask_id).all())
            gain = 12.0 if (self.sharp[i] or known_before) else 1.0
            logits[:, i, self.target[i]] = gain
        return logits


def test_block_generation_commits_confident_places_together_and_counts_steps():
    prompt = torch.tensor([[1, 2, 3, 4]])
    target = [1, 2, 3, 4] + [5, 6, 7, 8, 9, 10, 5, 6]
    sharp = [True] * 4 + [True, True, True, True, False, False, False, False]        # the first new block is easy, the second a chain
    obj = BlockDiffusionLM(Oracle(target, sharp), mask_id=11, block=4)
    out, steps = obj.generate(None, prompt, blocks=2, bound=0.05)
    assert out[0].tolist() == target
    # all four at once; then the place the prompt unlocks together with one uncertain place (a single uncertain place is an exact draw
    # from its marginal: the bound is on the entropies less the largest), and the remaining two likewise
    assert steps[0].tolist() == [1, 2]
    out, steps = obj.generate(None, prompt, blocks=2, bound=0.0)
    assert out[0].tolist() == target and steps[0].tolist() == [4, 4]
    out, steps = obj.generate(None, prompt, blocks=2, bound=0.05, max_steps=2)
    assert steps[0].tolist() == [1, 2] and int((out == 11).sum()) == 0           # the last allowed step commits what is left
    # a stop token ends a row: the rest of it is filled with the stop token
    stopper = BlockDiffusionLM(Oracle([1, 2, 3, 4, 5, 0, 7, 8, 9, 10, 5, 6], [True] * 12), mask_id=11, block=4)
    out, _ = stopper.generate(None, prompt, blocks=2, bound=1.0, stop_id=0)
    assert out[0].tolist() == [1, 2, 3, 4, 5, 0, 0, 0, 0, 0, 0, 0]


def test_masked_diffusion_trains_the_decoder_read_bidirectionally():
    """A pattern only the right-hand neighbour reveals: a causal decoder cannot fill it in, a bidirectional one can."""
    from dew_b200.models.causal_transformer import CausalTransformer, TransformerConfig
    from dew_b200.objectives.base import Step
    from dew_b200.objectives.discrete import MaskedDiffusionLM
    torch.manual_seed(0)
    V, MASK = 12, 11

    def batch(n):
        right = torch.randint(0, 5, (n, 4))
        rows = torch.stack([right + 5, right], 2).reshape(n, 8)          # each even place is its right neighbour plus five
        return {"tokens": rows}
    accuracy = {}
    for causal in (True, False):
        torch.manual_seed(1)
        model = CausalTransformer(TransformerConfig(vocab_size=V, emb_features=32, num_layers=2, num_heads=4, mlp_features=64, max_seq_len=8, qk_norm=False,
                                                    causal=causal), dtype=torch.float32)
        obj = MaskedDiffusionLM(model, mask_id=MASK)
        opt = torch.optim.Adam(model.parameters(), lr=3e-3)
        for i in range(150):
            stats, _ = obj.loss(None, batch(32), Step(step=i, key=i))
            opt.zero_grad()
            (stats.total / stats.mass).backward()
            opt.step()
        test = batch(64)["tokens"]
        hidden = test.clone()
        hidden[:, 0::2] = MASK                                           # hide the even places, keep what reveals them
        with torch.no_grad():
            out = model(hidden)
            out = out[0] if isinstance(out, tuple) else out
        accuracy[causal] = float((out.argmax(-1)[:, 0::2] == test[:, 0::2]).float().mean())
    assert accuracy[False] > 0.7 and accuracy[True] < 0.4, accuracy
