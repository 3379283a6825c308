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
