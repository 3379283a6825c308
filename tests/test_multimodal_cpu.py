"""Vision-language splicing, projectors, the log-mel front end and the audio encoder."""
import math

import pytest
import torch

import dew_b200 as dew
from dew_b200.models import CausalTransformer
from dew_b200.models.encoders import EncoderConfig, VisionTower
from dew_b200.models.multimodal import AudioEncoder, Projector, VisionLanguageModel, expand_placeholders, log_mel, mel_filters, splice
from dew_b200.objectives.lm import LMObjective


def _vlm(merge=1):
    torch.manual_seed(0)
    vision = VisionTower(EncoderConfig(features=32, layers=1, heads=2, mlp_features=64), image_size=16, patch=4)
    decoder = CausalTransformer(vocab_size=64, emb_features=48, num_layers=2, num_heads=2, head_dim=24, mlp_features=96, max_seq_len=64, qk_norm=False)
    return VisionLanguageModel(vision, decoder, image_token_id=63, vision_features=32, merge=merge)


def test_image_features_are_spliced_over_their_placeholders():
    m = _vlm()
    assert m.tokens_per_image(16) == 16
    row = expand_placeholders([1, 63, 2, 3], 63, 16)
    assert len(row) == 19 and row[1:17] == [63] * 16
    tokens = torch.tensor([row, row])
    images = torch.randn(2, 3, 16, 16)
    emb = m.embeddings(tokens, images)
    feats = m.image_features(images)
    assert feats.shape == (2, 16, 48) and torch.allclose(emb[:, 1:17], feats) and torch.equal(emb[:, 0], m.decoder.embed(tokens)[:, 0])
    logits = m(tokens, images)
    assert logits.shape == (2, 19, 64)
    # the text after the image depends on the image; the text before it does not (causal)
    other = m(tokens, torch.randn(2, 3, 16, 16))
    assert torch.allclose(other[:, 0], logits[:, 0], atol=1e-5) and not torch.allclose(other[:, 17:], logits[:, 17:], atol=1e-4)
    # without images it is the decoder alone
    text = torch.tensor([[1, 2, 3, 4]])
    assert torch.allclose(m(text), m.decoder(text))
    with pytest.raises(ValueError, match="placeholder"):
        m(torch.tensor([[1, 63, 2]]), images[:1])
    # gradients reach the projector and the decoder, not the frozen tower
    loss = logits.float().pow(2).mean()
    loss.backward()
    assert m.projector.fc1.weight.grad is not None and m.decoder.embed.weight.grad is not None
    assert all(p.grad is None for p in m.vision.parameters())
    merged = _vlm(merge=2)
    assert merged.tokens_per_image(16) == 4 and merged.image_features(images).shape == (2, 4, 48)
    p = Projector(8, 12, "linear", merge=2)
    x = torch.arange(2 * 16 * 8, dtype=torch.float32).reshape(2, 16, 8)
    folded = x.reshape(2, 2, 2, 2, 2, 8).permute(0, 1, 3, 2, 4, 5).reshape(2, 4, 32)
    assert torch.allclose(p(x), p.fc1(p.norm(folded)))
    assert torch.equal(splice(torch.zeros(1, 3, 2), torch.tensor([[5, 9, 9]]), 9, torch.ones(2, 2))[0], torch.tensor([[0.0, 0], [1, 1], [1, 1]]))


def test_a_vision_language_model_trains_through_the_lm_objective():
    m = _vlm()
    torch.manual_seed(1)
    # the caption's first token names the image's dominant channel: only the image can tell
    images, rows = [], []
    for i in range(32):
        c = i % 3
        img = torch.randn(3, 16, 16) * 0.1
        img[c] += 1.0
        images.append(img)
        rows.append(expand_placeholders([1, 63, 10 + c, 2], 63, 16))
    tokens, images = torch.tensor(rows), torch.stack(images)

    class Objective(LMObjective):
        def apply(self, variables, inputs, **kw):
            return self.model(inputs, images=self._images, **kw)
    obj = Objective(m, tokens.shape[1] - 1, pad_id=63)                      # the placeholders are not predicted
    obj._images = images
    tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    tr.fit([{"tokens": tokens}] * 60, steps=60, log_every=20)
    assert t.rows[-1]["loss"] < 0.5 * t.rows[0]["loss"]
    with torch.no_grad():
        pred = m(tokens, images)[:, 16].argmax(-1)                          # the position of the last image token predicts the class token
    assert float((pred == tokens[:, 17]).float().mean()) > 0.9


def test_log_mel_and_the_audio_encoder():
    bank = mel_filters(16000, 400, 80)
    assert bank.shape == (80, 201) and float(bank.min()) >= 0 and torch.all(bank.sum(1) > 0)
    peaks = bank.argmax(1)
    assert torch.all(peaks[1:] >= peaks[:-1])                               # centre frequencies rise with the filter index
    t = torch.arange(16000) / 16000
    low, high = torch.sin(2 * math.pi * 300 * t)[None], torch.sin(2 * math.pi * 3000 * t)[None]
    ml, mh = log_mel(low), log_mel(high)
    assert ml.shape == (1, 100, 80) and int(ml.mean(1).argmax()) < int(mh.mean(1).argmax())
    assert float(ml.max() - ml.min()) <= 2.0 + 1e-5                         # the 8-decade clamp, then / 4
    enc = AudioEncoder(n_mels=80, features=32, layers=1, heads=2, max_frames=64)
    mel = torch.cat([ml, mh])
    out, mask = enc(mel, lengths=torch.tensor([100, 60]))
    assert out.shape == (2, 50, 32) and mask.sum(1).tolist() == [50, 30] and enc.frames(100) == 50
    # padding frames do not change the real frames' outputs
    changed = mel.clone()
    changed[1, 60:] = 5.0
    out2, _ = enc(changed, lengths=torch.tensor([100, 60]))
    assert torch.allclose(out2[1, :29], out[1, :29], atol=1e-5)
