"""Text and vision towers (CLIP, SigLIP, ViT, DINOv2, T5) against the ``transformers`` implementations on random tiny models,
weights through ``dew_b200.interop.encoders``; the pipeline-style text conditioner on top of them."""
import pytest
import torch

from dew_b200.interop import encoders as E
from dew_b200.interop.conditioners import TextConditioner, TowerBinding, whitespace_tokenizer

T = pytest.importorskip("transformers")
SMALL = dict(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64)


def _random(model):
    torch.manual_seed(1)
    for p in model.parameters():
        if p.dim() == 1:                           # biases, norms and gains away from their neutral values
            p.data.add_(torch.randn_like(p) * 0.1)
    return model.float().eval()


@pytest.fixture(scope="module")
def inputs():
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(3, 99, (2, 16), generator=g)
    ids[:, 10] = 98
    return ids, torch.randn(2, 3, 32, 32, generator=g)


def test_clip_towers(inputs):
    ids, img = inputs
    cfg = T.CLIPConfig(text_config=dict(vocab_size=99, max_position_embeddings=16, eos_token_id=2, **SMALL),
                       vision_config=dict(image_size=32, patch_size=8, **SMALL), projection_dim=16)
    cfg._attn_implementation = "eager"
    m = _random(T.CLIPModel(cfg))
    with torch.no_grad():
        want_t, want_v = m.text_model(ids), m.vision_model(img)
    text, left_t = E.clip_text(cfg.text_config.to_dict(), m.state_dict(), dtype=torch.float32)
    vision, left_v = E.clip_vision(cfg.vision_config.to_dict(), m.state_dict(), dtype=torch.float32)
    assert [k for k in left_t if k.startswith("text_model.")] == [] and left_v == []
    with torch.no_grad():
        s, p = text(ids)
        tk, vp = vision(img)
        pen, _ = text(ids, None, -2)
        want_pen = m.text_model(ids, output_hidden_states=True).hidden_states[-2]
    assert torch.allclose(s, want_t.last_hidden_state, atol=1e-5) and torch.allclose(p, want_t.pooler_output, atol=1e-5)
    assert torch.allclose(tk, want_v.last_hidden_state, atol=1e-5) and torch.allclose(vp, want_v.pooler_output, atol=1e-5)
    assert torch.allclose(pen, want_pen, atol=1e-5)                  # the penultimate layer, as SDXL-style pipelines take it


def test_siglip_towers(inputs):
    ids, img = inputs
    cfg = T.SiglipConfig(text_config=dict(vocab_size=99, max_position_embeddings=16, **SMALL), vision_config=dict(image_size=32, patch_size=8, **SMALL))
    cfg._attn_implementation = "eager"
    m = _random(T.SiglipModel(cfg))
    with torch.no_grad():
        want_t, want_v = m.text_model(ids), m.vision_model(img)
    text, left_t = E.siglip_text(cfg.text_config.to_dict(), m.state_dict(), dtype=torch.float32)
    vision, left_v = E.siglip_vision(cfg.vision_config.to_dict(), m.state_dict(), dtype=torch.float32)
    assert left_t == [] and left_v == []
    with torch.no_grad():
        s, p = text(ids)
        tk, vp = vision(img)
    assert torch.allclose(s, want_t.last_hidden_state, atol=1e-5) and torch.allclose(p, want_t.pooler_output, atol=1e-5)
    assert torch.allclose(tk, want_v.last_hidden_state, atol=1e-5) and torch.allclose(vp, want_v.pooler_output, atol=1e-5)


def test_vit_and_dinov2(inputs):
    _, img = inputs
    vc = T.ViTConfig(image_size=32, patch_size=8, **SMALL)
    vc._attn_implementation = "eager"
    vm = _random(T.ViTModel(vc, add_pooling_layer=False))
    tower, left = E.vit(vc.to_dict(), vm.state_dict(), dtype=torch.float32)
    assert left == []
    with torch.no_grad():
        assert torch.allclose(tower(img)[0], vm(img).last_hidden_state, atol=1e-5)
    dc = T.Dinov2Config(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, mlp_ratio=2, image_size=32, patch_size=8)
    dc._attn_implementation = "eager"
    dm = _random(T.Dinov2Model(dc))
    tower, left = E.dinov2(dc.to_dict(), dm.state_dict(), dtype=torch.float32)
    assert left == []
    with torch.no_grad():
        tk, pooled = tower(img)
        want = dm(img)
    assert torch.allclose(tk, want.last_hidden_state, atol=1e-5) and torch.allclose(pooled, want.pooler_output, atol=1e-5)


@pytest.mark.parametrize("proj", ["gated-gelu", "relu"])
def test_t5_encoder(inputs, proj):
    ids, _ = inputs
    tc = T.T5Config(vocab_size=99, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=4, feed_forward_proj=proj)
    tm = _random(T.T5EncoderModel(tc))
    mask = torch.ones(2, 16, dtype=torch.long)
    mask[1, 12:] = 0
    enc, left = E.t5_encoder(tc.to_dict(), tm.state_dict(), dtype=torch.float32)
    assert left == []
    with torch.no_grad():
        got, want = enc(ids, mask), tm(ids, attention_mask=mask).last_hidden_state
    assert torch.allclose(got[mask.bool()], want[mask.bool()], atol=2e-5)


def test_text_conditioner_combines_towers():
    from dew_b200.models.encoders import EncoderConfig, T5Encoder, TextTower
    torch.manual_seed(0)
    clip_a = TextTower(EncoderConfig(32, 2, 4, 64, "quick_gelu", causal=True), 200, 16, pool="eos").eval()
    clip_b = TextTower(EncoderConfig(48, 2, 4, 96, "gelu", causal=True), 200, 16, pool="eos").eval()
    t5 = T5Encoder(200, 64, 2, 4, 16, 128).eval()
    tok = whitespace_tokenizer(200)
    prompts = ["a red fox jumps", "two boats"]
    # SDXL style: penultimate states side by side, pooled from the second tower only
    sdxl = TextConditioner([TowerBinding(clip_a, tok, 16, layer=-2, use_pooled=False), TowerBinding(clip_b, tok, 16, layer=-2)])
    out = sdxl(prompts, negative=[""])
    assert out["context"].shape == (2, 16, 80) and out["pooled"].shape == (2, 48)
    assert out["uncond_context"].shape == (2, 16, 80) and not torch.equal(out["context"], out["uncond_context"])
    # SD3 style: CLIP states padded to T5's width and joined along the sequence; both pooled vectors
    sd3 = TextConditioner([TowerBinding(clip_a, tok, 16), TowerBinding(clip_b, tok, 16), TowerBinding(t5, tok, 24, use_pooled=False, masked=True)],
                          combine="sequence", context_width=64)
    out = sd3(prompts)
    assert out["context"].shape == (2, 16 + 16 + 24, 64) and out["pooled"].shape == (2, 80)
    assert torch.all(out["context"][:, :16, 32:] == 0)            # the narrower tower's states are zero-padded
