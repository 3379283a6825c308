"""Latent-diffusion checkpoints: both public FLUX layouts round-trip through the key maps, the autoencoder reads legacy names,
and a pipeline assembles from a component directory."""
import json
import os

import pytest
import torch
from safetensors.torch import save_file

from dew_b200.interop.diffusion import (autoencoder_kl_from_components, flux_config_from_original, flux_from_components, flux_from_original,
                                        flux_to_components, flux_to_original, load_pipeline)
from dew_b200.models.latent_autoencoders import AutoencoderKL
from dew_b200.models.latent_backbones import RectifiedFlowTransformer


def _flux(**kw):
    torch.manual_seed(0)
    m = RectifiedFlowTransformer(emb_features=64, num_heads=2, double_layers=2, single_layers=2, text_features=32, pooled_features=24, guidance_embed=True, **kw)
    with torch.no_grad():
        for p in m.parameters():                                       # the zero-initialised layers too, so a swapped tensor shows
            p.copy_(torch.randn_like(p) * 0.05)
    return m


def _same_function(a, b):
    x, t = torch.randn(2, 8, 8, 16), torch.tensor([0.3, 0.8])
    ctx = {"text": torch.randn(2, 5, 32), "pooled": torch.randn(2, 24), "guidance": torch.tensor([3.5, 1.0])}
    with torch.no_grad():
        return torch.allclose(a(x, t, ctx), b(x, t, ctx), atol=1e-5)


def test_flux_original_layout_round_trips():
    m = _flux()
    tensors = flux_to_original(m)
    assert {"img_in.weight", "time_in.in_layer.weight", "vector_in.out_layer.bias", "guidance_in.in_layer.weight", "double_blocks.1.img_attn.qkv.weight",
            "double_blocks.0.txt_attn.norm.key_norm.scale", "double_blocks.0.img_mod.lin.bias", "double_blocks.1.txt_mlp.2.weight",
            "single_blocks.1.linear1.weight", "single_blocks.0.norm.query_norm.scale", "single_blocks.0.modulation.lin.weight",
            "final_layer.adaLN_modulation.1.weight", "final_layer.linear.bias"} <= set(tensors)
    assert len(tensors) == len(m.state_dict())
    cfg = flux_config_from_original(tensors)
    assert cfg["emb_features"] == 64 and cfg["num_heads"] == 2 and cfg["double_layers"] == 2 and cfg["single_layers"] == 2 and cfg["guidance_embed"]
    assert cfg["text_features"] == 32 and cfg["pooled_features"] == 24 and cfg["input_channels"] == 16 and cfg["mlp_ratio"] == 4.0
    back = flux_from_original(tensors)
    assert _same_function(m, back)
    del tensors["single_blocks.1.linear2.bias"]
    with pytest.raises(KeyError):
        flux_from_original(tensors, cfg)
    assert flux_from_original(tensors, cfg, strict=False) is not None


def test_flux_component_layout_splits_fuses_and_swaps():
    m = _flux()
    tensors = flux_to_components(m)
    assert {"x_embedder.weight", "context_embedder.bias", "time_text_embed.timestep_embedder.linear_1.weight", "time_text_embed.guidance_embedder.linear_2.bias",
            "time_text_embed.text_embedder.linear_1.weight", "transformer_blocks.0.attn.to_q.weight", "transformer_blocks.1.attn.add_v_proj.bias",
            "transformer_blocks.0.attn.norm_added_k.weight", "transformer_blocks.0.norm1_context.linear.weight", "transformer_blocks.0.ff.net.0.proj.weight",
            "transformer_blocks.0.ff_context.net.2.bias", "transformer_blocks.0.attn.to_add_out.weight", "single_transformer_blocks.1.proj_mlp.weight",
            "single_transformer_blocks.0.attn.to_k.bias", "single_transformer_blocks.0.proj_out.weight", "single_transformer_blocks.0.norm.linear.weight",
            "norm_out.linear.weight", "proj_out.bias"} <= set(tensors)
    sd = m.state_dict()
    assert torch.equal(tensors["transformer_blocks.0.attn.to_k.weight"], sd["double_blocks.0.img_qkv.weight"][64:128])
    assert torch.equal(tensors["single_transformer_blocks.0.proj_mlp.weight"], sd["single_blocks.0.linear1.weight"][192:])
    # the final modulation is stored (scale, shift) there and (shift, scale) here
    assert torch.equal(tensors["norm_out.linear.weight"][:64], sd["final_mod.weight"][64:]) and torch.equal(tensors["norm_out.linear.bias"][64:], sd["final_mod.bias"][:64])
    config = {"num_attention_heads": 2, "attention_head_dim": 32, "in_channels": 64, "num_layers": 2, "num_single_layers": 2, "joint_attention_dim": 32,
              "pooled_projection_dim": 24, "guidance_embeds": True, "patch_size": 1}
    back = flux_from_components(config, tensors)
    assert _same_function(m, back)
    # and the two layouts describe the same weights
    assert _same_function(flux_from_original(flux_to_original(back)), m)


def test_autoencoder_reads_legacy_attention_names_and_a_pipeline_assembles(tmp_path):
    torch.manual_seed(0)
    ae = AutoencoderKL.flux(block_out_channels=(32, 64), layers_per_block=1, norm_groups=8)
    legacy = {}
    for k, v in ae.state_dict().items():
        for new, old in (("to_q", "query"), ("to_k", "key"), ("to_v", "value"), ("to_out.0", "proj_attn")):
            if f"attentions.0.{new}." in k:
                k = k.replace(f"attentions.0.{new}.", f"attentions.0.{old}.")
                v = v[:, :, None, None] if v.dim() == 2 else v               # the first releases stored 1 x 1 convolutions
        legacy[k] = v.clone()
    config = {"in_channels": 3, "latent_channels": 16, "block_out_channels": [32, 64], "layers_per_block": 1, "norm_num_groups": 8,
              "scaling_factor": 0.3611, "shift_factor": 0.1159, "use_quant_conv": False}
    back = autoencoder_kl_from_components(config, legacy)
    x = torch.rand(1, 16, 16, 3) * 2 - 1
    with torch.no_grad():
        assert torch.allclose(back.encode(x), ae.encode(x), atol=1e-6) and back.normalization.shift == 0.1159
    # a component directory: model_index.json, one folder per component, the transformer's weights in two shards
    flux = _flux()
    root = tmp_path / "pipe"
    for name in ("transformer", "vae", "scheduler"):
        (root / name).mkdir(parents=True)
    (root / "model_index.json").write_text(json.dumps({"_class_name": "FluxPipeline", "_diffusers_version": "0.30.0",
                                                      "transformer": ["diffusers", "FluxTransformer2DModel"], "vae": ["diffusers", "AutoencoderKL"],
                                                      "scheduler": ["diffusers", "FlowMatchEulerDiscreteScheduler"], "tokenizer": ["transformers", "CLIPTokenizer"],
                                                      "image_encoder": [None, None]}))
    (root / "transformer" / "config.json").write_text(json.dumps({"_class_name": "FluxTransformer2DModel", "num_attention_heads": 2, "attention_head_dim": 32,
                                                                  "in_channels": 64, "num_layers": 2, "num_single_layers": 2, "joint_attention_dim": 32,
                                                                  "pooled_projection_dim": 24, "guidance_embeds": True}))
    tensors = {k: v.contiguous() for k, v in flux_to_components(flux).items()}
    names = sorted(tensors)
    shards = {"diffusion_pytorch_model-00001-of-00002.safetensors": names[: len(names) // 2], "diffusion_pytorch_model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for fname, keys in shards.items():
        save_file({k: tensors[k] for k in keys}, str(root / "transformer" / fname))
    (root / "transformer" / "diffusion_pytorch_model.safetensors.index.json").write_text(json.dumps({"weight_map": {k: f for f, ks in shards.items() for k in ks}}))
    (root / "vae" / "config.json").write_text(json.dumps({"_class_name": "AutoencoderKL", **config}))
    save_file({k: v.contiguous() for k, v in ae.state_dict().items()}, str(root / "vae" / "diffusion_pytorch_model.safetensors"))
    (root / "scheduler" / "scheduler_config.json").write_text(json.dumps({"shift": 3.0, "use_dynamic_shifting": True, "base_shift": 0.5, "max_shift": 1.15}))
    pipe = load_pipeline(str(root))
    assert pipe.kind == "FluxPipeline" and _same_function(pipe.transformer, flux)
    with torch.no_grad():
        assert torch.allclose(pipe.vae.decode(pipe.vae.encode(x)), ae.decode(ae.encode(x)), atol=1e-5)
    assert pipe.solver_settings()["shift"] == 3.0 and pipe.solver_settings()["dynamic"] and pipe.solver_settings()["max_tokens"] == 4096
    only = load_pipeline(str(root), components=["vae"])
    assert only.transformer is None and only.vae is not None
    (root / "model_index.json").write_text(json.dumps({"_class_name": "X", "unet": ["diffusers", "UNet2DConditionModel"]}))
    (root / "unet").mkdir()
    with pytest.raises(ValueError, match="does not build"):
        load_pipeline(str(root))
