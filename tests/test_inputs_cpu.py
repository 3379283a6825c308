"""Condition encoders, their records and dispatch, the CLIP image transform and inpainting conditions."""
import numpy as np
import pytest
import torch

from dew_b200.inputs import CharTable, CLIPImageTransform, Condition, ConditionEncoder, Field, InputSpec, TowerEncoder, encode_conditions, latent_image_conditions
from dew_b200.inputs.diffusion import blend_known
from dew_b200.inputs.encoders import char_codes


def test_char_table_encodes_masks_pools_and_rebuilds_from_its_record():
    tok = char_codes(["ab", "", "a" * 50], tokens=8, vocab=258)
    assert tok["tokens"].shape == (3, 8) and tok["tokens"][0, :3].tolist() == [1, 2 + ord("a") % 256, 2 + ord("b") % 256]
    assert tok["mask"].sum(1).tolist() == [3, 1, 8]
    enc = CharTable(features=16, tokens=8, seed=3)
    ctx = enc.encode(**enc.tokenize(["ab", ""]))
    assert ctx["text"].shape == (2, 8, 16) and torch.all(ctx["text"][0, 3:] == 0) and ctx["pooled"].shape == (2, 16)
    assert torch.allclose(ctx["pooled"][0], ctx["text"][0, :3].mean(0))
    again = ConditionEncoder.bound(enc.record())
    assert isinstance(again, CharTable) and torch.equal(again.table, enc.table) and again.record() == enc.record()
    assert torch.equal(enc.null(2)["tokens"], enc.tokenize(["", ""])["tokens"])
    with pytest.raises(KeyError):
        ConditionEncoder.bound({"class": "nope"})


def test_encode_conditions_dispatches_by_encoder_kind():
    enc = CharTable(features=8, tokens=6)
    spec = InputSpec(Field("sample", (8, 8, 3)), {"textcontext": Condition(Field("caption", (6,)), encoder=enc),
                                                  "label": Condition(Field("class", ()), encoder=lambda v: v.float() * 2),
                                                  "absent": Condition(Field("nothing", ()))})
    tok = enc.tokenize(["a cat", "a dog"])
    out = encode_conditions(spec.conditions, {"caption": tok["tokens"], "caption_mask": tok["mask"], "class": torch.tensor([1, 2])})
    assert set(out) == {"textcontext", "label"} and out["textcontext"]["text"].shape == (2, 6, 8) and out["label"].tolist() == [2.0, 4.0]
    from_text = encode_conditions(spec.conditions, {"caption_text": ["a cat", "a dog"]})
    assert torch.equal(from_text["textcontext"]["text"], out["textcontext"]["text"])

    class Tower(torch.nn.Module):
        def __init__(self):
            super().__init__(); self.emb = torch.nn.Embedding(300, 8)
        def forward(self, ids, key_mask=None):
            h = self.emb(ids)
            return h, h.mean(1)
    tower = TowerEncoder(Tower(), lambda texts: char_codes(texts, 6, 258))
    ctx = tower.encode(**tower.tokenize(["hi"]))
    assert ctx["text"].shape == (1, 6, 8) and ctx["pooled"].shape == (1, 8) and not ctx["text"].requires_grad
    assert all(not p.requires_grad for p in tower.tower.parameters())


def test_clip_image_transform_matches_the_published_steps():
    g = torch.Generator().manual_seed(0)
    img = torch.randint(0, 256, (2, 300, 400, 3), generator=g, dtype=torch.uint8)
    out = CLIPImageTransform(224)(img)
    assert out.shape == (2, 3, 224, 224) and out.dtype == torch.float32
    # an image already at the target size is only cropped (nothing) and normalised
    small = torch.randint(0, 256, (1, 224, 224, 3), generator=g, dtype=torch.uint8)
    want = (small.permute(0, 3, 1, 2).float() / 255 - torch.tensor([0.48145466, 0.4578275, 0.40821073]).view(1, 3, 1, 1)) / torch.tensor([0.26862954, 0.26130258, 0.27577711]).view(1, 3, 1, 1)
    assert torch.allclose(CLIPImageTransform(224)(small), want, atol=1e-6)
    # against PIL's bicubic resize of the shorter side + centre crop (the processor's own steps), up to interpolation differences
    from PIL import Image
    pil = Image.fromarray(img[0].numpy()).resize((round(400 * 224 / 300), 224), Image.BICUBIC)
    left = (pil.size[0] - 224) // 2
    ref = torch.from_numpy(np.asarray(pil.crop((left, 0, left + 224, 224)), dtype=np.float32)).permute(2, 0, 1) / 255
    got = out[0] * torch.tensor([0.26862954, 0.26130258, 0.27577711]).view(3, 1, 1) + torch.tensor([0.48145466, 0.4578275, 0.40821073]).view(3, 1, 1)
    assert float((got - ref).abs().mean()) < 0.02


def test_inpainting_conditions_and_known_region_blend():
    class AE:
        def encode(self, x):
            return torch.nn.functional.avg_pool2d(x.permute(0, 3, 1, 2), 4).permute(0, 2, 3, 1)
    pixels = torch.ones(1, 16, 16, 3)
    mask = torch.zeros(1, 16, 16)
    mask[:, :8] = 1                                                         # repaint the top half
    c = latent_image_conditions(pixels, mask, AE())
    assert c["mask"].shape == (1, 4, 4, 1) and c["masked_image"].shape == (1, 4, 4, 3)
    assert torch.all(c["mask"][0, :2] == 1) and torch.all(c["mask"][0, 2:] == 0)
    assert torch.all(c["masked_image"][0, :2] == 0) and torch.all(c["masked_image"][0, 2:] == 1)
    lat, orig, noise = torch.full((1, 4, 4, 3), 5.0), torch.ones(1, 4, 4, 3), torch.zeros(1, 4, 4, 3)
    out = blend_known(lat, orig, c["mask"], noise, alpha=0.5, sigma=0.3)
    assert torch.all(out[0, :2] == 5.0) and torch.all(out[0, 2:] == 0.5)
