"""Mamba and Mamba-2 releases load into ``CausalTransformer`` (blocks of one mixer and no MLP) and give the logits ``transformers`` gives;
they write back name for name."""
import warnings

import pytest
import torch

from dew_b200.interop.recurrent import export_recurrent_state, load_recurrent_state, read_recurrent_config, write_recurrent_config
from dew_b200.models.causal_transformer import CausalTransformer, TransformerConfig

CASES = {
    "mamba": dict(model_type="mamba", vocab_size=96, hidden_size=64, state_size=8, num_hidden_layers=2, expand=2, conv_kernel=4, time_step_rank=4),
    "mamba2": dict(model_type="mamba2", vocab_size=96, hidden_size=64, state_size=16, num_hidden_layers=2, expand=2, head_dim=16, num_heads=8, n_groups=2,
                   conv_kernel=4, chunk_size=32),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_state_space_release_matches_transformers(name):
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    cfg = transformers.AutoConfig.for_model(**CASES[name])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        hf = transformers.AutoModelForCausalLM.from_config(cfg).float().eval()
    for n, p in hf.named_parameters():
        if p.dim() == 1 and "A_log" not in n:
            p.data.add_(torch.randn_like(p) * 0.1)
    d = cfg.to_dict()
    ours = CausalTransformer(read_recurrent_config(d), dtype=torch.float32).eval()
    assert all(layer.mlp is None and layer.post_norm is None for layer in ours.layers)
    assert load_recurrent_state(ours, dict(hf.state_dict())) == []
    tokens = torch.randint(0, 96, (2, 40))
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("ignore")
        want = hf(tokens).logits
        got = ours(tokens)
        got = got[0] if isinstance(got, tuple) else got
    assert float((got - want).abs().max()) <= 2e-5 * max(1.0, float(want.abs().max())), float((got - want).abs().max())
    back = export_recurrent_state(ours)
    theirs = {k: v for k, v in hf.state_dict().items() if not (k == "lm_head.weight" and ours.head is None)}
    assert sorted(back) == sorted(theirs)
    for k, v in theirs.items():
        assert torch.equal(back[k], v), k
    again = read_recurrent_config(write_recurrent_config(ours.config))
    assert again.mixer_options == ours.config.mixer_options and again.kinds() == ours.config.kinds()


def test_layers_of_one_sub_layer():
    """A mixer-only layer and an MLP-only layer in turn make the same function as one ordinary layer."""
    torch.manual_seed(0)
    base = dict(vocab_size=50, emb_features=32, num_heads=4, mlp_features=64, max_seq_len=32, qk_norm=False)
    whole = CausalTransformer(TransformerConfig(num_layers=1, **base), dtype=torch.float32).eval()
    split = CausalTransformer(TransformerConfig(num_layers=2, layer_types=("attention", "none"), layer_mlp=(False, True), **base), dtype=torch.float32).eval()
    with torch.no_grad():
        split.embed.weight.copy_(whole.embed.weight)
        split.final_norm.weight.copy_(whole.final_norm.weight)
        a, b, w = split.layers[0], split.layers[1], whole.layers[0]
        a.input_norm.weight.copy_(w.input_norm.weight), a.mixer.load_state_dict(w.mixer.state_dict())
        b.input_norm.weight.copy_(w.post_norm.weight), b.mlp.load_state_dict(w.mlp.state_dict())
    tokens = torch.randint(0, 50, (2, 12))
    with torch.no_grad():
        x, y = whole(tokens), split(tokens)
    x, y = (x[0] if isinstance(x, tuple) else x), (y[0] if isinstance(y, tuple) else y)
    assert torch.allclose(x, y, atol=1e-6)
    with pytest.raises(ValueError, match="neither"):
        CausalTransformer(TransformerConfig(num_layers=1, layer_types=("none",), layer_mlp=(False,), **base))
