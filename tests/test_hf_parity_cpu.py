"""Logits parity with Hugging Face implementations on tiny random models (weights travel through the interop loader)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from dew_b200.interop.hf import Pretrained  # noqa: E402


def _compare(hf, tmp_path, vocab, atol=2e-5):
    hf = hf.eval()
    hf.save_pretrained(tmp_path, safe_serialization=True)
    mine = Pretrained.load(tmp_path).eval()
    tok = torch.randint(0, vocab, (2, 19), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        a, b = hf(tok).logits.float(), mine(tok).float()
    assert float((a - b).abs().max()) < atol * max(1.0, float(a.abs().max())), float((a - b).abs().max())
    return mine


def test_llama_parity_and_round_trip(tmp_path):
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-6, tie_word_embeddings=False,
                                   rope_parameters={"rope_theta": 500000.0, "rope_type": "default"})
    mine = _compare(transformers.LlamaForCausalLM(cfg), tmp_path / "llama", 128)
    assert mine.config.rope_theta == 500000.0                 # read from the nested rotary settings
    # and back: the exported directory loads in transformers with the same logits
    Pretrained.save(mine, tmp_path / "back")
    again = transformers.LlamaForCausalLM.from_pretrained(tmp_path / "back").eval()
    tok = torch.randint(0, 128, (1, 11))
    with torch.no_grad():
        assert torch.allclose(again(tok).logits.float(), mine(tok).float(), atol=2e-5)


def test_qwen3_parity_with_qk_norm(tmp_path):
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(vocab_size=128, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=16, max_position_embeddings=64, tie_word_embeddings=False)
    hf = transformers.Qwen3ForCausalLM(cfg)
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "q_norm" in n or "k_norm" in n:
                p.add_(0.1 * torch.randn_like(p))
    _compare(hf, tmp_path / "qwen3", 128)


def test_mixtral_parity(tmp_path):
    torch.manual_seed(0)
    cfg = transformers.MixtralConfig(vocab_size=128, hidden_size=64, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                                     num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2, max_position_embeddings=64,
                                     sliding_window=None, tie_word_embeddings=False)
    mine = _compare(transformers.MixtralForCausalLM(cfg), tmp_path / "mixtral", 128, atol=5e-5)
    assert mine.config.mixture.experts == 4 and mine.config.mixture.top_k == 2


def test_qwen3_moe_parity_and_export(tmp_path):
    torch.manual_seed(0)
    cfg = transformers.Qwen3MoeConfig(vocab_size=128, hidden_size=64, intermediate_size=112, moe_intermediate_size=32, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_experts=4, num_experts_per_tok=2,
                                      norm_topk_prob=True, max_position_embeddings=64, tie_word_embeddings=False, decoder_sparse_step=1,
                                      mlp_only_layers=[])
    mine = _compare(transformers.Qwen3MoeForCausalLM(cfg), tmp_path / "q3moe", 128, atol=5e-5)
    Pretrained.save(mine, tmp_path / "back", architecture="Qwen3MoeForCausalLM")
    again = transformers.Qwen3MoeForCausalLM.from_pretrained(tmp_path / "back").eval()
    tok = torch.randint(0, 128, (1, 13))
    with torch.no_grad():
        assert torch.allclose(again(tok).logits.float(), mine(tok).float(), atol=5e-5)


def test_greedy_generation_matches_transformers(tmp_path):
    from dew_b200.sampling.text import Sampling, generate
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=64, tie_word_embeddings=False, eos_token_id=None, bos_token_id=None)
    hf = transformers.LlamaForCausalLM(cfg).eval()
    hf.save_pretrained(tmp_path / "m", safe_serialization=True)
    mine = Pretrained.load(tmp_path / "m").eval()
    prompt = [5, 17, 99, 3, 42]
    with torch.no_grad():
        want = hf.generate(torch.tensor([prompt]), max_new_tokens=10, do_sample=False, pad_token_id=0)[0, len(prompt):].tolist()
    got = generate(mine, None, [prompt], 10, sampling=Sampling(temperature=0.0))
    assert [int(t) for t in got.new_tokens(0)] == want


def test_gated_delta_net_layer_matches_qwen3_next():
    """The gated-delta-rule mixer (short conv, l2-normalised q / k, decay and write gates, chunked delta rule, gated RMSNorm)
    against the Qwen3-Next layer of transformers, weights copied through the interop."""
    import warnings
    from dew_b200.interop.hf import load_gated_delta_net
    from dew_b200.nn.linear_attention import GatedDeltaNet
    try:
        from transformers.models.qwen3_next import modeling_qwen3_next as Q
    except Exception:
        pytest.skip("this transformers has no Qwen3-Next")
    torch.manual_seed(0)
    cfg = transformers.Qwen3NextConfig(vocab_size=64, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                       num_key_value_heads=2, head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4,
                                       linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4, num_experts=0,
                                       max_position_embeddings=128, layer_types=["linear_attention", "full_attention"])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        hf = Q.Qwen3NextGatedDeltaNet(cfg, 0).eval()
    with torch.no_grad():
        hf.A_log.copy_(torch.randn(4) * 0.5)
        hf.dt_bias.copy_(torch.randn(4) * 0.5)
        hf.norm.weight.copy_(1 + 0.1 * torch.randn(16))
    mine = GatedDeltaNet(64, num_k_heads=2, num_v_heads=4, head_k_dim=16, head_v_dim=16, conv_size=4, norm_eps=cfg.rms_norm_eps).eval()
    load_gated_delta_net(mine, hf.state_dict())
    for T in (24, 100):                                       # one chunk and several
        x = torch.randn(2, T, 64)
        with torch.no_grad():
            a, b = hf(x), mine(x)
        assert float((a - b).abs().max()) < 2e-5 * max(1.0, float(a.abs().max())), (T, float((a - b).abs().max()))


def test_mamba2_layer_matches_transformers():
    import warnings
    from dew_b200.interop.hf import load_mamba2
    from dew_b200.nn.mamba2 import Mamba2
    from transformers.models.mamba2 import modeling_mamba2 as M
    torch.manual_seed(0)
    cfg = transformers.Mamba2Config(vocab_size=64, hidden_size=64, state_size=16, num_hidden_layers=1, expand=2, head_dim=16, num_heads=8, n_groups=1,
                                    conv_kernel=4, chunk_size=32, use_bias=False, use_conv_bias=True, rms_norm=True)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        hf = M.Mamba2Mixer(cfg, 0).eval()
    with torch.no_grad():
        hf.A_log.copy_(torch.log(torch.rand(8) * 4 + 1))
        hf.dt_bias.copy_(torch.randn(8) * 0.5)
        hf.D.copy_(torch.randn(8))
        hf.norm.weight.copy_(1 + 0.1 * torch.randn(128))
        hf.conv1d.bias.copy_(torch.randn(160) * 0.1)
    mine = Mamba2(64, state_dim=16, head_dim=16, norm_eps=cfg.layer_norm_epsilon).eval()
    load_mamba2(mine, hf.state_dict())
    for T in (24, 80):
        x = torch.randn(2, T, 64)
        with torch.no_grad():
            a, b = hf(x), mine(x)
        assert float((a - b).abs().max()) < 2e-5 * max(1.0, float(a.abs().max())), (T, float((a - b).abs().max()))


def test_mamba1_layer_matches_transformers():
    import warnings
    from dew_b200.nn.mamba import Mamba
    from transformers.models.mamba import modeling_mamba as M
    torch.manual_seed(0)
    cfg = transformers.MambaConfig(vocab_size=64, hidden_size=64, state_size=8, num_hidden_layers=1, expand=2, conv_kernel=4, time_step_rank=4,
                                   use_bias=False, use_conv_bias=True)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        hf = M.MambaMixer(cfg, 0).eval()
    mine = Mamba(64, state_dim=8, expand=2, conv_size=4, dt_rank=4).eval()
    with torch.no_grad():
        hf.A_log.copy_(torch.log(torch.rand(128, 8) * 4 + 0.5))
        hf.D.copy_(torch.randn(128))
        hf.conv1d.bias.copy_(torch.randn(128) * 0.1)
        hf.dt_proj.bias.copy_(torch.randn(128) * 0.3)
        sd, named = hf.state_dict(), dict(mine.named_parameters())
        for k in ("A_log", "D", "in_proj.weight", "x_proj.weight", "dt_proj.weight", "dt_proj.bias", "out_proj.weight"):
            named[k].copy_(sd[k])
        mine.conv.weight.copy_(sd["conv1d.weight"].reshape(128, 4))
        mine.conv.bias.copy_(sd["conv1d.bias"])
    for T in (20, 70):
        x = torch.randn(2, T, 64)
        with torch.no_grad():
            a, b = hf(x), mine(x)
        assert float((a - b).abs().max()) < 1e-5, (T, float((a - b).abs().max()))


def test_multi_head_latent_attention_matches_deepseek_v3():
    import warnings
    from dew_b200 import ops
    from dew_b200.interop.hf import load_mla
    from dew_b200.nn.mla import MultiHeadLatentAttention
    from transformers.models.deepseek_v3 import modeling_deepseek_v3 as D
    torch.manual_seed(0)
    cfg = transformers.DeepseekV3Config(vocab_size=64, hidden_size=64, intermediate_size=96, num_hidden_layers=1, num_attention_heads=4,
                                        num_key_value_heads=4, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
                                        v_head_dim=16, max_position_embeddings=64, rope_scaling=None, n_routed_experts=4, first_k_dense_replace=1)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        hf = D.DeepseekV3Attention(cfg, 0).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.copy_(1 + 0.1 * torch.randn_like(p))
    mine = MultiHeadLatentAttention(64, 4, kv_latent=16, q_latent=24, nope_dim=16, rope_dim=8, v_dim=16, norm_eps=cfg.rms_norm_eps).eval()
    load_mla(mine, hf.state_dict())
    B, T = 2, 12
    x = torch.randn(B, T, 64)
    mask = torch.full((T, T), float("-inf")).triu(1)[None, None]
    inv = 1.0 / (10000.0 ** (torch.arange(0, 8, 2).float() / 8))
    ang = torch.arange(T).float()[:, None] * inv[None]
    emb = torch.cat([ang, ang], -1)
    cos, sin = ops.rope_tables(64, 8, 10000.0, "cpu", None)
    with torch.no_grad():
        a = hf(x, position_embeddings=(emb.cos()[None].expand(B, T, 8), emb.sin()[None].expand(B, T, 8)), attention_mask=mask)[0]
        b = mine(x, cos, sin)
    assert float((a - b).abs().max()) < 1e-5, float((a - b).abs().max())


def test_group_limited_router_matches_deepseek_v3():
    import warnings
    from dew_b200.models.causal_transformer import Mixture
    from dew_b200.nn.moe import Router
    from transformers.models.deepseek_v3 import modeling_deepseek_v3 as D
    torch.manual_seed(0)
    cfg = transformers.DeepseekV3Config(vocab_size=64, hidden_size=32, intermediate_size=48, moe_intermediate_size=16, num_hidden_layers=1,
                                        num_attention_heads=2, num_key_value_heads=2, n_routed_experts=16, num_experts_per_tok=4, n_group=4,
                                        topk_group=2, norm_topk_prob=True, routed_scaling_factor=2.5, q_lora_rank=8, kv_lora_rank=8,
                                        qk_nope_head_dim=8, qk_rope_head_dim=8, v_head_dim=8, first_k_dense_replace=0)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        hf = D.DeepseekV3MoE(cfg).eval()
    with torch.no_grad():
        hf.gate.weight.normal_(0, 0.5)
        hf.gate.e_score_correction_bias.normal_(0, 0.1)
    mix = Mixture(experts=16, top_k=4, score_function="sigmoid", norm_topk_prob=True, scaling=2.5, bias=True, groups=4, topk_groups=2)
    mine = Router(32, mix)
    with torch.no_grad():
        mine.weight.copy_(hf.gate.weight)
        mine.expert_bias.copy_(hf.gate.e_score_correction_bias)
    x = torch.randn(40, 32)
    with torch.no_grad():
        logits = hf.gate(x)
        out = hf.route_tokens_to_experts(logits) if hasattr(hf, "route_tokens_to_experts") else logits
        ids_hf, w_hf = out
        w, ids, _ = mine(x)
    order_a, order_b = ids_hf.sort(-1), ids.sort(-1)
    assert torch.equal(order_a.values, order_b.values)
    assert torch.allclose(w_hf.gather(-1, order_a.indices).float(), w.gather(-1, order_b.indices), atol=1e-5)


def test_sparse_mlp_matches_deepseek_v3_moe_block():
    """Routed experts under group-limited sigmoid routing plus the shared experts, against transformers' block."""
    import warnings
    from dew_b200.models.causal_transformer import Mixture
    from dew_b200.nn.moe import SparseMLP
    from transformers.models.deepseek_v3 import modeling_deepseek_v3 as D
    torch.manual_seed(0)
    cfg = transformers.DeepseekV3Config(vocab_size=64, hidden_size=32, intermediate_size=48, moe_intermediate_size=16, num_hidden_layers=1,
                                        num_attention_heads=2, num_key_value_heads=2, n_routed_experts=8, num_experts_per_tok=3, n_group=4,
                                        topk_group=2, norm_topk_prob=True, routed_scaling_factor=2.5, n_shared_experts=2, q_lora_rank=8,
                                        kv_lora_rank=8, qk_nope_head_dim=8, qk_rope_head_dim=8, v_head_dim=8, first_k_dense_replace=0)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        hf = D.DeepseekV3MoE(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.2)
    sd = hf.state_dict()
    if "experts.gate_up_proj" not in sd:
        pytest.skip("this transformers stores the experts one module each")
    mix = Mixture(experts=8, top_k=3, score_function="sigmoid", norm_topk_prob=True, scaling=2.5, bias=True, groups=4, topk_groups=2,
                  expert_features=16, shared_features=32)
    mine = SparseMLP(32, mix, 48).eval()
    with torch.no_grad():
        mine.router.weight.copy_(sd["gate.weight"])
        mine.router.expert_bias.copy_(sd["gate.e_score_correction_bias"])
        mine.experts.gate_up.copy_(sd["experts.gate_up_proj"])
        mine.experts.down.copy_(sd["experts.down_proj"])
        mine.shared.gate_up_proj.weight.copy_(torch.cat([sd["shared_experts.gate_proj.weight"], sd["shared_experts.up_proj.weight"]], 0))
        mine.shared.down_proj.weight.copy_(sd["shared_experts.down_proj.weight"])
    x = torch.randn(2, 9, 32)
    with torch.no_grad():
        a, b = hf(x), mine(x)
    assert float((a - b).abs().max()) < 2e-5 * max(1.0, float(a.abs().max()))
