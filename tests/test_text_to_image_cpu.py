"""The text-to-image task over a tiny class / text conditioned DiT."""
import pytest
import torch

from dew_b200.diffusion import presets
from dew_b200.inference.images import ImageRequest, ImageSettings, Images, TextToImage, serve
from dew_b200.inputs import Condition, Field, InputSpec
from dew_b200.models.dit import SimpleDiT
from dew_b200.objectives.diffusion import DiffusionObjective
from dew_b200.sampling import CFG, Euler


class _Bag:
    """A toy text encoder: byte histogram -> 8 features per prompt."""

    def __call__(self, prompts):
        out = torch.zeros(len(prompts), 8)
        for i, p in enumerate(prompts):
            for ch in p.encode():
                out[i, ch % 8] += 1.0
        return out / out.sum(1, keepdim=True).clamp_min(1)


def _task():
    torch.manual_seed(0)
    model = SimpleDiT(patch_size=4, emb_features=32, num_layers=2, num_heads=2, text_features=8)
    with torch.no_grad():
        for p in model.parameters():
            p.add_(0.05 * torch.randn_like(p))
    inputs = InputSpec(Field("sample", (16, 16, 3)), {"text": Condition(Field("text", ()), encoder=_Bag())})
    obj = DiffusionObjective(model, presets.Flow(), inputs, ema_decay=None, solver=Euler(), guidance=CFG(2.0), steps=4)
    return TextToImage.from_objective(obj)


def test_prompts_to_images_reproducible_and_guided():
    task = _task()
    a = task(["a red flower", "a blue sky"], key=5)
    assert isinstance(a, Images) and a.decoded.shape == (2, 16, 16, 3) and float(a.decoded.abs().max()) <= 1.0
    assert a.pixels().dtype == torch.uint8 and len(a.pil()) == 2
    assert torch.equal(task(["a red flower", "a blue sky"], key=5).decoded, a.decoded)          # same key, same images
    assert not torch.equal(task(["a red flower", "a blue sky"], key=6).decoded, a.decoded)
    # guidance changes the walk; scale 1 equals the unguided conditional walk
    unguided = task(["a red flower", "a blue sky"], key=5, guidance=None)
    one = task(["a red flower", "a blue sky"], key=5, guidance=1.0)
    assert torch.allclose(unguided.decoded, one.decoded, atol=1e-5) and not torch.allclose(unguided.decoded, a.decoded, atol=1e-4)
    # a different prompt draws a different image from the same prior
    b = task(["a green field", "a blue sky"], key=5)
    assert not torch.allclose(a.decoded[0], b.decoded[0], atol=1e-5) and torch.allclose(a.decoded[1], b.decoded[1], atol=1e-5)


def test_settings_steps_latents_and_requests():
    task = _task()
    seen = []
    out = task(["x"], key=1, steps=3, on_step=lambda i, x: seen.append(tuple(x.shape)))
    assert len(seen) == 3 and seen[0] == (1, 16, 16, 3) and out.decoded.shape == (1, 16, 16, 3)
    raw = task(["x"], key=1, settings=ImageSettings(steps=3, decode=False))
    assert raw.decoded is None and raw.latents.shape == (1, 16, 16, 3)
    with pytest.raises(ValueError):
        raw.pixels()
    with pytest.raises(ValueError):
        ImageSettings(steps=0)
    with pytest.raises(KeyError):
        task(conditions={"label": torch.tensor([1])})
    answers = serve(task, [ImageRequest(["x"], key=1, settings=ImageSettings(steps=3)), ImageRequest(["y", "z"], key=2)])
    assert torch.allclose(answers[0].decoded, out.decoded) and answers[1].decoded.shape[0] == 2
    moved = task.bind({"params": {}})
    assert moved.variables == {"params": {}} and task.variables is None
