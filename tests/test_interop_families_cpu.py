"""Decoder families: every family's release layout loads into ``CausalTransformer`` and gives the logits the
``transformers`` implementation of that family gives (fp32, eager attention); round trips through the on-disk layout;
sharded files, fp8 block storage, keys nothing read."""
import json

import pytest
import torch

from dew_b200.interop.families import FAMILIES, export_state, family_of, load_state, read_config
from dew_b200.interop.hf import Pretrained
from dew_b200.interop.release import GenerationConfig, Release, dequantize_blocks, quantize_blocks, save_release
from dew_b200.models.causal_transformer import CausalTransformer

COMMON = dict(vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              intermediate_size=128, max_position_embeddings=64)
CASES = {
    "llama": dict(model_type="llama", head_dim=16, **COMMON),
    "mistral": dict(model_type="mistral", head_dim=16, sliding_window=8, **COMMON),
    "qwen2": dict(model_type="qwen2", **COMMON),
    "qwen3": dict(model_type="qwen3", head_dim=16, **COMMON),
    "gemma": dict(model_type="gemma", head_dim=16, **COMMON),
    "gemma2": dict(model_type="gemma2", head_dim=16, sliding_window=8, query_pre_attn_scalar=24, **COMMON),
    "phi3": dict(model_type="phi3", pad_token_id=0, **COMMON),
    "olmo2": dict(model_type="olmo2", **COMMON),
    # (unscaled rotary: the installed transformers gives OLMo-3 one table for all layers, the release's own modelling code one per layer kind)
    "olmo3": dict(model_type="olmo3", sliding_window=8, layer_types=["sliding_attention", "full_attention"], **COMMON),
    "smollm3": dict(model_type="smollm3", no_rope_layers=[1, 0], pad_token_id=0, **COMMON),
    "gemma3": dict(model_type="gemma3_text", head_dim=16, sliding_window=8, query_pre_attn_scalar=24,
                   layer_types=["sliding_attention", "full_attention"],
                   rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 1000.0},
                                    "full_attention": {"rope_type": "linear", "rope_theta": 50000.0, "factor": 2.0}}, **COMMON),
    "granite": dict(model_type="granite", embedding_multiplier=6.0, attention_multiplier=0.1, residual_multiplier=0.3, logits_scaling=4.0, **COMMON),
    "deepseek_v3": dict(model_type="deepseek_v3", vocab_size=96, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
                        intermediate_size=128, max_position_embeddings=64, moe_intermediate_size=32, n_routed_experts=8, num_experts_per_tok=3,
                        n_group=4, topk_group=2, n_shared_experts=2, routed_scaling_factor=2.5, first_k_dense_replace=1, q_lora_rank=24,
                        kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, pad_token_id=0,
                        rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0, "original_max_position_embeddings": 16,
                                         "beta_fast": 32.0, "beta_slow": 1.0, "mscale": 1.0, "mscale_all_dim": 1.0}),
    "glm4": dict(model_type="glm4", head_dim=16, pad_token_id=0, **COMMON),
    "gpt_oss": dict(model_type="gpt_oss", vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                    intermediate_size=32, num_local_experts=4, num_experts_per_tok=2, max_position_embeddings=64, sliding_window=8,
                    layer_types=["sliding_attention", "full_attention"],
                    rope_parameters={"rope_type": "yarn", "rope_theta": 150000.0, "factor": 4.0, "original_max_position_embeddings": 16,
                                     "beta_fast": 32.0, "beta_slow": 1.0, "truncate": False}),
    "qwen2_moe": dict(model_type="qwen2_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=48, **COMMON),
    "qwen3_next": dict(model_type="qwen3_next", vocab_size=96, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       intermediate_size=128, moe_intermediate_size=32, shared_expert_intermediate_size=48, num_experts=4, num_experts_per_tok=2,
                       max_position_embeddings=64, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16,
                       linear_conv_kernel_dim=4, full_attention_interval=4),
    "mixtral": dict(model_type="mixtral", num_local_experts=4, num_experts_per_tok=2, **COMMON),
    "qwen3_moe": dict(model_type="qwen3_moe", head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                      norm_topk_prob=True, **COMMON),
}


def _logits(model, tokens):
    y = model(tokens)
    return y[0] if isinstance(y, tuple) else y


@pytest.mark.parametrize("name", sorted(CASES))
def test_family_matches_transformers(name, tmp_path):
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    cfg = transformers.AutoConfig.for_model(**CASES[name])
    cfg._attn_implementation = "eager"
    hf = transformers.AutoModelForCausalLM.from_config(cfg).float().eval()
    for n, p in hf.named_parameters():
        if p.dim() == 1 or n.endswith("_bias"):   # norms away from one, biases away from zero
            p.data.add_(torch.randn_like(p) * 0.1)
    d = cfg.to_dict()
    fam = family_of(d)
    assert fam.name == name
    ours = CausalTransformer(read_config(d), dtype=torch.float32).eval()
    assert load_state(ours, dict(hf.state_dict()), fam) == []
    tokens = torch.randint(0, 96, (2, 24))
    with torch.no_grad():
        want = hf(tokens).logits
        got = _logits(ours, tokens)
    assert float((got - want).abs().max()) <= 2e-6 * max(1.0, float(want.abs().max()))
    # and back: the exported tensors are the release's, name for name
    back = export_state(ours, fam)
    theirs = {k: v for k, v in hf.state_dict().items() if not (k == "lm_head.weight" and ours.head is None)}
    if fam.experts is None:                   # (sparse families: the module keeps experts stacked, the files hold one tensor per expert)
        assert sorted(back) == sorted(theirs)
    for k, v in theirs.items():
        if k in back:
            assert torch.allclose(back[k], v, atol=1e-6), k
    # through the directory layout, in shards
    Pretrained.save(ours, tmp_path, family=name, max_shard_bytes=60_000, generation=GenerationConfig(eos_token_id=[1, 2], temperature=0.7))
    assert (tmp_path / "model.safetensors.index.json").exists()
    again = Pretrained.load(tmp_path, dtype=torch.float32).eval()
    assert again.family == name and again.generation_config.stop_ids() == (1, 2)
    with torch.no_grad():
        assert torch.equal(_logits(again, tokens), got)


def test_unread_keys_raise():
    torch.manual_seed(0)
    cfg = read_config(CASES["llama"])
    m = CausalTransformer(cfg, dtype=torch.float32)
    state = export_state(m, FAMILIES["llama"])
    state["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    with pytest.raises(KeyError, match="not read"):
        load_state(m, state, FAMILIES["llama"])
    assert load_state(m, state, FAMILIES["llama"], strict=False) == ["model.layers.0.self_attn.q_proj.bias"]
    with pytest.raises(KeyError, match="no decoder family"):
        family_of({"model_type": "bert", "architectures": ["BertModel"]})


def test_release_reads_lazily_and_dequantizes_fp8_blocks(tmp_path):
    torch.manual_seed(0)
    w = torch.randn(200, 300)
    q, s = quantize_blocks(w, (128, 128))
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 3)
    deq = dequantize_blocks(q, s, (128, 128), torch.float32)
    assert float((deq - w).abs().max()) <= float(w.abs().max()) * 2 ** -4        # e4m3: 3 mantissa bits
    tensors = {"model.layers.0.mlp.down_proj.weight": w, "model.embed_tokens.weight": torch.randn(50, 300),
               "model.layers.1.mlp.down_proj.weight": torch.randn(200, 300)}
    names = save_release(tensors, {"model_type": "llama"}, tmp_path, max_shard_bytes=100_000, fp8_blocks=(128, 128))
    assert len(names) >= 2
    rel = Release(tmp_path, dtype=torch.float32)
    assert rel.config["quantization_config"]["weight_block_size"] == [128, 128]
    assert sorted(rel) == sorted(tensors)                  # the scales belong to their weights, not to the mapping
    assert rel.opened == []
    got = rel["model.layers.0.mlp.down_proj.weight"]
    assert len(rel.opened) >= 1 and len(rel.opened) < len(names) + 1
    assert torch.equal(got, deq)
    assert torch.equal(rel["model.embed_tokens.weight"], tensors["model.embed_tokens.weight"])     # skipped names stay as they are
    raw = Release(tmp_path, dequantize=False)
    assert raw["model.layers.0.mlp.down_proj.weight"].dtype == torch.float8_e4m3fn
    assert "model.layers.0.mlp.down_proj.weight_scale_inv" in raw


def test_rotary_scalings_match_transformers():
    transformers = pytest.importorskip("transformers")
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    from dew_b200 import ops
    yarns = [dict(rope_type="yarn", rope_theta=10000.0, factor=8.0, original_max_position_embeddings=16, beta_fast=32.0, beta_slow=1.0),
             dict(rope_type="yarn", rope_theta=50000.0, factor=8.0, original_max_position_embeddings=16, mscale=0.7, mscale_all_dim=1.0, truncate=False)]
    for rp in yarns:
        cfg = transformers.LlamaConfig(hidden_size=64, num_attention_heads=4, head_dim=16, max_position_embeddings=128, rope_parameters=dict(rp))
        inv, gain = ROPE_INIT_FUNCTIONS["yarn"](cfg, "cpu")
        ang = torch.outer(torch.arange(128).double(), inv.double())
        cos, sin = ops.rope_tables(128, 16, rp["rope_theta"], "cpu", {k: v for k, v in rp.items() if k != "rope_theta"})
        assert float((cos - (ang.cos() * gain).float()).abs().max()) < 5e-6 and float((sin - (ang.sin() * gain).float()).abs().max()) < 5e-6
    rp = dict(rope_type="longrope", rope_theta=10000.0, short_factor=[1.0 + 0.1 * i for i in range(8)], long_factor=[2.0 + 0.3 * i for i in range(8)],
              original_max_position_embeddings=32)
    cfg = transformers.Phi3Config(hidden_size=64, num_attention_heads=4, max_position_embeddings=128, original_max_position_embeddings=32,
                                  rope_parameters=dict(rp), pad_token_id=0)
    inv, gain = ROPE_INIT_FUNCTIONS["longrope"](cfg, "cpu", seq_len=100)
    ang = torch.outer(torch.arange(128).double(), inv.double())
    cos, _ = ops.rope_tables(128, 16, 10000.0, "cpu", {k: v for k, v in rp.items() if k != "rope_theta"})
    assert float((cos - (ang.cos() * gain).float()).abs().max()) < 5e-6
    short, _ = ops.rope_tables(32, 16, 10000.0, "cpu", {k: v for k, v in rp.items() if k != "rope_theta"})      # within the original context: the short set
    want = torch.outer(torch.arange(32).double(), 1.0 / (torch.tensor(rp["short_factor"]).double() * 10000.0 ** (torch.arange(0, 16, 2).double() / 16))).cos()
    assert float((short - want.float()).abs().max()) < 1e-6
    rp = dict(rope_type="dynamic", rope_theta=10000.0, factor=2.0)
    cfg = transformers.LlamaConfig(hidden_size=64, num_attention_heads=4, head_dim=16, max_position_embeddings=32, rope_parameters=dict(rp))
    inv, gain = ROPE_INIT_FUNCTIONS["dynamic"](cfg, "cpu", seq_len=128)
    ang = torch.outer(torch.arange(128).double(), inv.double())
    cos, _ = ops.rope_tables(128, 16, 10000.0, "cpu", {"rope_type": "dynamic", "factor": 2.0, "original_max_position_embeddings": 32})
    assert float((cos - (ang.cos() * gain).float()).abs().max()) < 5e-6
    with pytest.raises(ValueError, match="not built"):
        ops.rope_tables(32, 16, 10000.0, "cpu", {"rope_type": "su", "factor": 2.0})


def test_dream_is_qwen2_read_bidirectionally():
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    cfg = transformers.AutoConfig.for_model(**CASES["qwen2"])
    cfg._attn_implementation = "eager"
    hf = transformers.AutoModelForCausalLM.from_config(cfg).float().eval()
    d = dict(cfg.to_dict(), model_type="Dream", architectures=["DreamModel"])
    fam = family_of(d)
    assert fam.name == "dream"
    config = read_config(d)
    assert config.causal is False
    ours = CausalTransformer(config, dtype=torch.float32).eval()
    assert load_state(ours, dict(hf.state_dict()), fam) == []
    tokens = torch.randint(0, 96, (2, 12))
    everything = torch.zeros(2, 1, 12, 12)                                   # an additive mask that hides nothing
    with torch.no_grad():
        want = hf(tokens, attention_mask=everything).logits
        got = _logits(ours, tokens)
        causal = hf(tokens).logits
    assert float((got - want).abs().max()) <= 2e-6 * max(1.0, float(want.abs().max()))
    assert float((got - causal).abs().max()) > 1e-3
    later = tokens.clone()
    later[:, -1] = (later[:, -1] + 1) % 96
    with torch.no_grad():
        assert not torch.allclose(_logits(ours, later)[:, 0], got[:, 0])       # the first place reads the last
