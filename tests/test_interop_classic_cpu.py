"""The older decoder families load into ``ClassicDecoder`` and give the logits ``transformers`` gives (fp32, eager attention); they write
back name for name; generation with the per-layer cache agrees with the full forward."""
import pytest
import torch

from dew_b200.interop.classic import CLASSIC, classic_family_of, export_classic_state, load_classic, load_classic_state, read_classic_config
from dew_b200.models.classic_decoder import ClassicDecoder, alibi_slopes

CASES = {
    "gpt2": dict(model_type="gpt2", vocab_size=96, n_embd=64, n_layer=2, n_head=4, n_positions=64),
    "gpt_bigcode": dict(model_type="gpt_bigcode", vocab_size=96, n_embd=64, n_layer=2, n_head=4, n_positions=64),
    "gpt_neox": dict(model_type="gpt_neox", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                     max_position_embeddings=64, rotary_pct=0.25),
    "gpt_neox_sequential": dict(model_type="gpt_neox", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                                max_position_embeddings=64, rotary_pct=0.5, use_parallel_residual=False),
    "falcon": dict(model_type="falcon", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=64),
    "falcon_grouped": dict(model_type="falcon", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_kv_heads=2,
                           new_decoder_architecture=True, max_position_embeddings=64),
    "falcon_grouped_one_norm": dict(model_type="falcon", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_kv_heads=2,
                                    new_decoder_architecture=True, num_ln_in_parallel_attn=1, max_position_embeddings=64),
    "gptj": dict(model_type="gptj", vocab_size=96, n_embd=64, n_layer=2, n_head=4, n_positions=64, rotary_dim=8),
    "phi": dict(model_type="phi", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128, max_position_embeddings=64),
    "opt": dict(model_type="opt", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, ffn_dim=128, max_position_embeddings=64,
                word_embed_proj_dim=64),
    "opt_post_norm": dict(model_type="opt", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, ffn_dim=128, max_position_embeddings=64,
                          word_embed_proj_dim=32, do_layer_norm_before=False),
    "bloom": dict(model_type="bloom", vocab_size=96, hidden_size=64, n_layer=2, n_head=4),
    "starcoder2": dict(model_type="starcoder2", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=128, max_position_embeddings=64, sliding_window=8),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_classic_family_matches_transformers(name):
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    cfg = transformers.AutoConfig.for_model(**CASES[name])
    cfg._attn_implementation = "eager"
    hf = transformers.AutoModelForCausalLM.from_config(cfg).float().eval()
    for p in hf.parameters():
        if p.dim() == 1:                      # norms away from one, biases away from zero
            p.data.add_(torch.randn_like(p) * 0.1)
    d = cfg.to_dict()
    fam = classic_family_of(d)
    assert fam.name == (name if name.startswith("falcon_grouped") else CASES[name]["model_type"])
    ours = ClassicDecoder(read_classic_config(d), dtype=torch.float32).eval()
    assert load_classic_state(ours, dict(hf.state_dict()), fam) == []
    tokens = torch.randint(3, 96, (2, 24))
    with torch.no_grad():
        want = hf(tokens).logits
        got = ours(tokens)
    assert float((got - want).abs().max()) <= 3e-6 * max(1.0, float(want.abs().max())), float((got - want).abs().max())
    back = export_classic_state(ours, fam)
    theirs = {k: v for k, v in hf.state_dict().items() if not (k == fam.names["head"] + ".weight" and ours.head is None)
              and not k.endswith((".attn.bias", ".attn.masked_bias", ".attention.bias", ".attention.masked_bias", "rotary_emb.inv_freq"))}
    assert sorted(back) == sorted(theirs)
    for k, v in theirs.items():
        assert torch.equal(back[k], v), k
    # the cache: a prefix, then one token at a time
    with torch.no_grad():
        cache = ours.new_cache()
        first = ours(tokens[:, :10], cache=cache)
        steps = [ours(tokens[:, t:t + 1], cache=cache) for t in range(10, 24)]
    stepped = torch.cat([first] + steps, 1)
    assert float((stepped - got).abs().max()) <= 2e-5 * max(1.0, float(got.abs().max()))


def test_alibi_slopes_and_generation():
    s = alibi_slopes(8)
    assert torch.allclose(s, torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    s12 = alibi_slopes(12)                               # not a power of two: eight, then every other term of sixteen's
    assert torch.allclose(s12[:8], s) and torch.allclose(s12[8:], torch.tensor([2.0 ** -(0.5 * (2 * i + 1)) for i in range(4)]))
    torch.manual_seed(0)
    m = ClassicDecoder(vocab_size=50, emb_features=32, num_layers=2, num_heads=4, max_seq_len=32, positions="alibi").eval()
    prompt = torch.randint(0, 50, (2, 5))
    out = m.generate(prompt, 6)
    assert out.shape == (2, 11) and torch.equal(out[:, :5], prompt)
    with torch.no_grad():                                # greedy: every new token is the argmax of the full forward at its position
        full = m(out[:, :-1])
    assert torch.equal(full[:, 4:].argmax(-1), out[:, 5:])


def test_unknown_and_unbuilt_layouts_raise():
    with pytest.raises(KeyError, match="no classic decoder family"):
        classic_family_of({"model_type": "llama"})
    with pytest.raises(NotImplementedError, match="not ALiBi"):
        read_classic_config(dict(CASES["falcon"], alibi=True))
    torch.manual_seed(0)
    m = ClassicDecoder(read_classic_config(CASES["gpt2"]), dtype=torch.float32)
    state = export_classic_state(m, CLASSIC["gpt2"])
    state["transformer.h.0.attn.extra.weight"] = torch.zeros(3)
    with pytest.raises(KeyError, match="not read"):
        load_classic_state(m, state, CLASSIC["gpt2"])
    again = load_classic(CASES["gpt2"], export_classic_state(m, CLASSIC["gpt2"]), dtype=torch.float32)
    tokens = torch.randint(0, 96, (1, 9))
    with torch.no_grad():
        assert torch.equal(again(tokens), m(tokens))


def test_pretrained_loads_a_saved_directory(tmp_path):
    transformers = pytest.importorskip("transformers")
    from dew_b200.interop.hf import Pretrained
    torch.manual_seed(0)
    cfg = transformers.AutoConfig.for_model(**CASES["gpt_neox"])
    cfg._attn_implementation = "eager"
    hf = transformers.AutoModelForCausalLM.from_config(cfg).float().eval()
    hf.save_pretrained(tmp_path, safe_serialization=True)
    ours = Pretrained.load(tmp_path, dtype=torch.float32).eval()
    assert ours.family == "gpt_neox" and ours.unread_keys == []
    tokens = torch.randint(0, 96, (1, 12))
    with torch.no_grad():
        want, got = hf(tokens).logits, ours(tokens)
    assert float((got - want).abs().max()) <= 3e-6 * max(1.0, float(want.abs().max()))
