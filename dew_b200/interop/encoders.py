"""Published text and vision towers -> ``dew_b200.models.encoders``: configuration translation and weight-name mapping for CLIP
(text, vision), SigLIP (text, vision with its attention-pooling probe), ViT, DINOv2 and T5's encoder.  Every loader returns the
release's keys it did not read (empty for a complete mapping), so a silent partial load cannot happen.

Reference: src/dew/interop/text_encoders.py (CLIP / T5 towers), encoders.py, conditioners.py, src/dew/nn/vision/*.
"""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Tuple

import torch

from ..models.encoders import EncoderConfig, T5Encoder, TextTower, VisionTower


class _Reader:
    def __init__(self, tensors: Mapping[str, torch.Tensor], prefix: str = ""):
        self.t, self.prefix, self.read = tensors, prefix, set()

    def __call__(self, key: str) -> torch.Tensor:
        self.read.add(self.prefix + key)
        return self.t[self.prefix + key]

    def has(self, key: str) -> bool:
        return self.prefix + key in self.t

    def unread(self, ignore: Tuple[str, ...] = ("position_ids", "mask_token")) -> List[str]:
        return sorted(k for k in self.t if k.startswith(self.prefix) and k not in self.read and not any(i in k for i in ignore))


def _put(p: torch.Tensor, t: torch.Tensor) -> None:
    if tuple(p.shape) != tuple(t.shape):
        t = t.reshape(p.shape)
    with torch.no_grad():
        p.copy_(t.to(p.dtype))


def _linear(lin, get: _Reader, name: str) -> None:
    _put(lin.weight, get(name + ".weight"))
    if lin.bias is not None:
        _put(lin.bias, get(name + ".bias"))


def _norm(norm, get: _Reader, name: str) -> None:
    _put(norm.weight, get(name + ".weight"))
    _put(norm.bias, get(name + ".bias"))


def _clip_layers(encoder, get: _Reader, base: str) -> None:
    for i, blk in enumerate(encoder.blocks):
        pre = f"{base}.{i}."
        _norm(blk.norm1, get, pre + "layer_norm1")
        _norm(blk.norm2, get, pre + "layer_norm2")
        for ours, theirs in (("q_proj", "q_proj"), ("k_proj", "k_proj"), ("v_proj", "v_proj"), ("out_proj", "out_proj")):
            _linear(getattr(blk.attn, ours), get, pre + "self_attn." + theirs)
        _linear(blk.fc1, get, pre + "mlp.fc1")
        _linear(blk.fc2, get, pre + "mlp.fc2")


def _encoder_config(c: Mapping[str, Any], causal: bool = False, layer_scale: bool = False) -> EncoderConfig:
    act = c.get("hidden_act", "gelu")
    return EncoderConfig(features=c["hidden_size"], layers=c["num_hidden_layers"], heads=c["num_attention_heads"],
                         mlp_features=c.get("intermediate_size") or int(c["hidden_size"] * c.get("mlp_ratio", 4)), activation=act,
                         norm_eps=c.get("layer_norm_eps", 1e-5), causal=causal, layer_scale=layer_scale)


# ------------------------------------------------------------------------------------------------ CLIP
def clip_text(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], dtype=None, device=None) -> Tuple[TextTower, List[str]]:
    eos = config.get("eos_token_id")
    tower = TextTower(_encoder_config(config, causal=True), config["vocab_size"], config.get("max_position_embeddings", 77), pool="eos",
                      eos_token_id=None if eos in (None, 2) else eos, dtype=dtype, device=device)      # (id 2: the legacy configs, argmax rule)
    get = _Reader(tensors, "text_model.")
    _put(tower.token.weight, get("embeddings.token_embedding.weight"))
    _put(tower.position.weight, get("embeddings.position_embedding.weight"))
    _clip_layers(tower.encoder, get, "encoder.layers")
    _norm(tower.final_norm, get, "final_layer_norm")
    return tower, get.unread()


def clip_vision(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], dtype=None, device=None) -> Tuple[VisionTower, List[str]]:
    tower = VisionTower(_encoder_config(config), config["image_size"], config["patch_size"], config.get("num_channels", 3), class_token=True,
                        pre_norm=True, pool="class", patch_bias=False, norm_tokens=False, dtype=dtype, device=device)
    get = _Reader(tensors, "vision_model.")
    _put(tower.class_token, get("embeddings.class_embedding"))
    _put(tower.patch_embed.weight, get("embeddings.patch_embedding.weight"))
    _put(tower.position, get("embeddings.position_embedding.weight"))
    _norm(tower.pre_norm, get, "pre_layrnorm")
    _clip_layers(tower.encoder, get, "encoder.layers")
    _norm(tower.post_norm, get, "post_layernorm")
    return tower, get.unread()


# ------------------------------------------------------------------------------------------------ SigLIP
def siglip_vision(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], dtype=None, device=None) -> Tuple[VisionTower, List[str]]:
    tower = VisionTower(_encoder_config({**config, "layer_norm_eps": config.get("layer_norm_eps", 1e-6)}), config["image_size"], config["patch_size"],
                        config.get("num_channels", 3), class_token=False, pool="probe", dtype=dtype, device=device)
    get = _Reader(tensors, "vision_model.")
    _put(tower.patch_embed.weight, get("embeddings.patch_embedding.weight"))
    _put(tower.patch_embed.bias, get("embeddings.patch_embedding.bias"))
    _put(tower.position, get("embeddings.position_embedding.weight"))
    _clip_layers(tower.encoder, get, "encoder.layers")
    _norm(tower.post_norm, get, "post_layernorm")
    _put(tower.probe, get("head.probe"))
    _put(tower.probe_attn.in_proj_weight, get("head.attention.in_proj_weight"))
    _put(tower.probe_attn.in_proj_bias, get("head.attention.in_proj_bias"))
    _linear(tower.probe_attn.out_proj, get, "head.attention.out_proj")
    _norm(tower.probe_norm, get, "head.layernorm")
    _linear(tower.probe_fc1, get, "head.mlp.fc1")
    _linear(tower.probe_fc2, get, "head.mlp.fc2")
    return tower, get.unread()


def siglip_text(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], dtype=None, device=None) -> Tuple[TextTower, List[str]]:
    tower = TextTower(_encoder_config({**config, "layer_norm_eps": config.get("layer_norm_eps", 1e-6)}), config["vocab_size"],
                      config.get("max_position_embeddings", 64), pool="last", head=True, dtype=dtype, device=device)
    get = _Reader(tensors, "text_model.")
    _put(tower.token.weight, get("embeddings.token_embedding.weight"))
    _put(tower.position.weight, get("embeddings.position_embedding.weight"))
    _clip_layers(tower.encoder, get, "encoder.layers")
    _norm(tower.final_norm, get, "final_layer_norm")
    _linear(tower.head, get, "head")
    return tower, get.unread()


# ------------------------------------------------------------------------------------------------ ViT / DINOv2
def vit(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], dtype=None, device=None) -> Tuple[VisionTower, List[str]]:
    """``ViTModel`` (pre-norm blocks named ``layernorm_before / after``); the pooler (dense + tanh on the class token) is not part of
    the tower: its two tensors come back as unread."""
    tower = VisionTower(_encoder_config({**config, "layer_norm_eps": config.get("layer_norm_eps", 1e-12)}), config["image_size"],
                        config["patch_size"], config.get("num_channels", 3), class_token=True, pool="class", dtype=dtype, device=device)
    get = _Reader(tensors)
    _put(tower.class_token, get("embeddings.cls_token"))
    _put(tower.position, get("embeddings.position_embeddings"))
    _put(tower.patch_embed.weight, get("embeddings.patch_embeddings.projection.weight"))
    _put(tower.patch_embed.bias, get("embeddings.patch_embeddings.projection.bias"))
    for i, blk in enumerate(tower.encoder.blocks):
        pre = f"encoder.layer.{i}."
        _norm(blk.norm1, get, pre + "layernorm_before")
        _norm(blk.norm2, get, pre + "layernorm_after")
        for ours, theirs in (("q_proj", "query"), ("k_proj", "key"), ("v_proj", "value")):
            _linear(getattr(blk.attn, ours), get, pre + "attention.attention." + theirs)
        _linear(blk.attn.out_proj, get, pre + "attention.output.dense")
        _linear(blk.fc1, get, pre + "intermediate.dense")
        _linear(blk.fc2, get, pre + "output.dense")
    _norm(tower.post_norm, get, "layernorm")
    return tower, get.unread()


def dinov2(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], dtype=None, device=None) -> Tuple[VisionTower, List[str]]:
    tower = VisionTower(_encoder_config({**config, "layer_norm_eps": config.get("layer_norm_eps", 1e-6)}, layer_scale=True), config["image_size"],
                        config["patch_size"], config.get("num_channels", 3), class_token=True, pool="class", dtype=dtype, device=device)
    get = _Reader(tensors)
    _put(tower.class_token, get("embeddings.cls_token"))
    _put(tower.position, get("embeddings.position_embeddings"))
    _put(tower.patch_embed.weight, get("embeddings.patch_embeddings.projection.weight"))
    _put(tower.patch_embed.bias, get("embeddings.patch_embeddings.projection.bias"))
    for i, blk in enumerate(tower.encoder.blocks):
        pre = f"encoder.layer.{i}."
        _norm(blk.norm1, get, pre + "norm1")
        _norm(blk.norm2, get, pre + "norm2")
        for ours, theirs in (("q_proj", "query"), ("k_proj", "key"), ("v_proj", "value")):
            _linear(getattr(blk.attn, ours), get, pre + "attention.attention." + theirs)
        _linear(blk.attn.out_proj, get, pre + "attention.output.dense")
        _linear(blk.fc1, get, pre + "mlp.fc1")
        _linear(blk.fc2, get, pre + "mlp.fc2")
        _put(blk.scale1, get(pre + "layer_scale1.lambda1"))
        _put(blk.scale2, get(pre + "layer_scale2.lambda1"))
    _norm(tower.post_norm, get, "layernorm")
    return tower, get.unread()


# ------------------------------------------------------------------------------------------------ T5
def t5_encoder(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], dtype=None, device=None) -> Tuple[T5Encoder, List[str]]:
    proj = config.get("feed_forward_proj", "relu")
    gated = proj.startswith("gated-")
    act = proj.split("-", 1)[1] if gated else proj
    enc = T5Encoder(config["vocab_size"], config["d_model"], config["num_layers"], config["num_heads"], config["d_kv"], config["d_ff"],
                    gated, {"gelu": "gelu_new"}.get(act, act), config.get("relative_attention_num_buckets", 32),
                    config.get("relative_attention_max_distance", 128), config.get("layer_norm_epsilon", 1e-6), dtype=dtype, device=device)
    get = _Reader(tensors)
    _put(enc.token.weight, get("shared.weight") if get.has("shared.weight") else get("encoder.embed_tokens.weight"))
    if get.has("encoder.embed_tokens.weight"):
        get.read.add("encoder.embed_tokens.weight")
    _put(enc.relative.weight, get("encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight"))
    for i, blk in enumerate(enc.blocks):
        pre = f"encoder.block.{i}.layer."
        _put(blk.norm1.weight, get(pre + "0.layer_norm.weight"))
        for ours, theirs in (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o")):
            _put(getattr(blk, ours).weight, get(pre + f"0.SelfAttention.{theirs}.weight"))
        _put(blk.norm2.weight, get(pre + "1.layer_norm.weight"))
        if gated:
            _put(blk.wi_0.weight, get(pre + "1.DenseReluDense.wi_0.weight"))
            _put(blk.wi_1.weight, get(pre + "1.DenseReluDense.wi_1.weight"))
        else:
            _put(blk.wi_0.weight, get(pre + "1.DenseReluDense.wi.weight"))
        _put(blk.wo.weight, get(pre + "1.DenseReluDense.wo.weight"))
    _put(enc.final_norm.weight, get("encoder.final_layer_norm.weight"))
    return enc, get.unread()
