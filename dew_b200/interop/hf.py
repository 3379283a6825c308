"""Hugging Face decoder checkpoints <-> ``CausalTransformer``: config translation, weight-name mapping (separate
q / k / v and gate / up projections are fused here), safetensors load and save.

Parity (capability): src/dew/interop (HF families <-> trees, safetensors), ``Pretrained.load``,
``PretrainedDecoder.from_model(...).save`` (docs/concepts/inference.md:100-118).  Families covered: Llama, Qwen2 /
Qwen3 (qk-norm), Mistral (window), Gemma-style (embed scaling) share this mapping.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any, Dict, Mapping, Optional

import torch

from ..checkpoints import tensors as TS
from ..models.causal_transformer import CausalTransformer, TransformerConfig


def config_from_hf(cfg: Mapping[str, Any]) -> TransformerConfig:
    heads = cfg["num_attention_heads"]
    arch = (cfg.get("architectures") or [""])[0].lower()
    # newer configs nest the rotary settings: {"rope_parameters": {"rope_theta": ..., "rope_type": "default" | "llama3" | ...}}
    rope = cfg.get("rope_parameters") or {}
    theta = rope.get("rope_theta", cfg.get("rope_theta", 10000.0))
    scaling = cfg.get("rope_scaling")
    if scaling is None and rope.get("rope_type", "default") != "default":
        scaling = {k: v for k, v in rope.items() if k != "rope_theta"}
    experts = cfg.get("num_local_experts") or cfg.get("num_experts")
    mixture = None
    if experts:
        from ..models.causal_transformer import Mixture
        # Mixtral renormalises the chosen weights always; Qwen-MoE says so in ``norm_topk_prob``
        mixture = Mixture(experts=int(experts), top_k=int(cfg.get("num_experts_per_tok", 2)),
                          expert_features=int(cfg.get("moe_intermediate_size") or cfg["intermediate_size"]),
                          norm_topk_prob=bool(cfg.get("norm_topk_prob", True)) if "mixtral" not in arch else True)
    return TransformerConfig(mixture=mixture, 
        vocab_size=cfg["vocab_size"], emb_features=cfg["hidden_size"], num_layers=cfg["num_hidden_layers"], num_heads=heads,
        num_kv_heads=cfg.get("num_key_value_heads", heads), head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
        mlp_features=cfg["intermediate_size"], max_seq_len=cfg.get("max_position_embeddings", 4096),
        rope_theta=theta, rope_scaling=scaling, norm_eps=cfg.get("rms_norm_eps", 1e-6),
        qk_norm="qwen3" in arch, tie_embeddings=cfg.get("tie_word_embeddings", False), window=cfg.get("sliding_window"),
        embed_scale="gemma" in arch)


def config_to_hf(c: TransformerConfig, architecture: str = "LlamaForCausalLM", dtype: str = "bfloat16") -> Dict[str, Any]:
    rope = {"rope_theta": c.rope_theta, "rope_type": "default"} if not c.rope_scaling else {"rope_theta": c.rope_theta, **c.rope_scaling}
    moe = {}
    if c.mixture is not None:
        m = c.mixture
        moe = {"num_experts": m.experts, "num_local_experts": m.experts, "num_experts_per_tok": m.top_k, "norm_topk_prob": m.norm_topk_prob,
               "moe_intermediate_size": m.expert_features or c.mlp_features, "decoder_sparse_step": 1, "mlp_only_layers": []}
    return {**moe, "rope_parameters": rope, "dtype": dtype, "architectures": [architecture], "vocab_size": c.vocab_size, "hidden_size": c.emb_features, "num_hidden_layers": c.num_layers,
            "num_attention_heads": c.num_heads, "num_key_value_heads": c.num_kv_heads or c.num_heads,
            "head_dim": c.head_dim or c.emb_features // c.num_heads, "intermediate_size": c.mlp_features,
            "max_position_embeddings": c.max_seq_len, "rope_theta": c.rope_theta, "rope_scaling": c.rope_scaling,
            "rms_norm_eps": c.norm_eps, "tie_word_embeddings": c.tie_embeddings, "hidden_act": "silu", "torch_dtype": dtype}


def from_hf_state(model: CausalTransformer, hf: Mapping[str, torch.Tensor]) -> None:
    """Copy HF tensors into ``model`` (fusing q|k|v and gate|up)."""
    def put(p, t):
        with torch.no_grad():
            p.copy_(t.to(p.dtype))
    put(model.embed.weight, hf["model.embed_tokens.weight"])
    for i, layer in enumerate(model.layers):
        pre = f"model.layers.{i}."
        put(layer.input_norm.weight, hf[pre + "input_layernorm.weight"])
        put(layer.post_norm.weight, hf[pre + "post_attention_layernorm.weight"])
        a = layer.mixer
        put(a.qkv_proj.weight, torch.cat([hf[pre + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0))
        put(a.o_proj.weight, hf[pre + "self_attn.o_proj.weight"])
        if a.q_norm is not None and pre + "self_attn.q_norm.weight" in hf:
            put(a.q_norm.weight, hf[pre + "self_attn.q_norm.weight"])
            put(a.k_norm.weight, hf[pre + "self_attn.k_norm.weight"])
        if getattr(layer, "sparse", False):
            _put_experts(put, layer.mlp, hf, pre)
            continue
        put(layer.mlp.gate_up_proj.weight, torch.cat([hf[pre + "mlp.gate_proj.weight"], hf[pre + "mlp.up_proj.weight"]], 0))
        put(layer.mlp.down_proj.weight, hf[pre + "mlp.down_proj.weight"])
    put(model.final_norm.weight, hf["model.norm.weight"])
    if model.head is not None:
        put(model.head.weight, hf.get("lm_head.weight", hf["model.embed_tokens.weight"]))


def _put_experts(put, mlp, hf: Mapping[str, torch.Tensor], pre: str) -> None:
    """A sparse layer's router and experts from either naming: stacked tensors (``mlp.gate.weight``, ``mlp.experts.gate_up_proj``
    ``[E, 2F, d]``, ``mlp.experts.down_proj`` ``[E, d, F]``) or one tensor per expert (Mixtral's ``block_sparse_moe.experts.j.w1 /
    w3 / w2``, Qwen-MoE's ``mlp.experts.j.gate_proj / up_proj / down_proj``)."""
    E = mlp.mix.experts
    for gate in ("mlp.gate.weight", "block_sparse_moe.gate.weight"):
        if pre + gate in hf:
            put(mlp.router.weight, hf[pre + gate])
            break
    else:
        raise KeyError(f"no router weight under {pre}")
    if pre + "mlp.experts.gate_up_proj" in hf:
        put(mlp.experts.gate_up, hf[pre + "mlp.experts.gate_up_proj"])
        put(mlp.experts.down, hf[pre + "mlp.experts.down_proj"])
        return
    if pre + "block_sparse_moe.experts.0.w1.weight" in hf:
        names = ("block_sparse_moe.experts.{}.w1.weight", "block_sparse_moe.experts.{}.w3.weight", "block_sparse_moe.experts.{}.w2.weight")
    else:
        names = ("mlp.experts.{}.gate_proj.weight", "mlp.experts.{}.up_proj.weight", "mlp.experts.{}.down_proj.weight")
    put(mlp.experts.gate_up, torch.stack([torch.cat([hf[pre + names[0].format(j)], hf[pre + names[1].format(j)]], 0) for j in range(E)]))
    put(mlp.experts.down, torch.stack([hf[pre + names[2].format(j)] for j in range(E)]))


def to_hf_state(model: CausalTransformer, architecture: str = "LlamaForCausalLM") -> Dict[str, torch.Tensor]:
    c = model.config
    H, Hkv = c.num_heads, c.num_kv_heads or c.num_heads
    D = c.head_dim or c.emb_features // c.num_heads
    out = {"model.embed_tokens.weight": model.embed.weight.detach(), "model.norm.weight": model.final_norm.weight.detach()}
    for i, layer in enumerate(model.layers):
        pre = f"model.layers.{i}."
        out[pre + "input_layernorm.weight"] = layer.input_norm.weight.detach()
        out[pre + "post_attention_layernorm.weight"] = layer.post_norm.weight.detach()
        w = layer.mixer.qkv_proj.weight.detach()
        out[pre + "self_attn.q_proj.weight"], out[pre + "self_attn.k_proj.weight"], out[pre + "self_attn.v_proj.weight"] = \
            w[: H * D], w[H * D:(H + Hkv) * D], w[(H + Hkv) * D:]
        out[pre + "self_attn.o_proj.weight"] = layer.mixer.o_proj.weight.detach()
        if layer.mixer.q_norm is not None:
            out[pre + "self_attn.q_norm.weight"] = layer.mixer.q_norm.weight.detach()
            out[pre + "self_attn.k_norm.weight"] = layer.mixer.k_norm.weight.detach()
        if getattr(layer, "sparse", False):
            # one tensor per expert, under the names the target family stores on disk
            gu_all, dn_all = layer.mlp.experts.gate_up.detach(), layer.mlp.experts.down.detach()
            Fe = gu_all.shape[1] // 2
            mixtral = "mixtral" in architecture.lower()
            out[pre + ("block_sparse_moe.gate.weight" if mixtral else "mlp.gate.weight")] = layer.mlp.router.weight.detach()
            for j in range(gu_all.shape[0]):
                base = pre + (f"block_sparse_moe.experts.{j}." if mixtral else f"mlp.experts.{j}.")
                g_n, u_n, d_n = ("w1", "w3", "w2") if mixtral else ("gate_proj", "up_proj", "down_proj")
                out[base + g_n + ".weight"], out[base + u_n + ".weight"], out[base + d_n + ".weight"] = gu_all[j, :Fe], gu_all[j, Fe:], dn_all[j]
            continue
        gu = layer.mlp.gate_up_proj.weight.detach()
        F_ = gu.shape[0] // 2
        out[pre + "mlp.gate_proj.weight"], out[pre + "mlp.up_proj.weight"] = gu[:F_], gu[F_:]
        out[pre + "mlp.down_proj.weight"] = layer.mlp.down_proj.weight.detach()
    if model.head is not None:
        out["lm_head.weight"] = model.head.weight.detach()
    return {k: v.contiguous() for k, v in out.items()}


class Pretrained:
    """Load / save a decoder in the layout its family's releases use (``interop.families`` picks the family from
    ``config.json``; ``interop.release`` reads one file or shards, de-quantising stored fp8 blocks)."""

    @staticmethod
    def load(directory: os.PathLike, dtype=None, device="cpu", strict: bool = True):
        """A ``CausalTransformer`` for the families of ``interop.families``; a ``ClassicDecoder`` for the older lineage of
        ``interop.classic`` (GPT-2, GPT-NeoX, Falcon, Phi, OPT, BLOOM, StarCoder2, GPTBigCode); Mamba and Mamba-2 releases through
        ``interop.recurrent``."""
        from .classic import CLASSIC, load_classic_state, read_classic_config
        from .families import family_of, load_state, read_config
        from .release import GenerationConfig, Release
        rel = Release(directory, dtype=dtype or torch.bfloat16)
        if str(rel.config.get("model_type") or "").lower() in CLASSIC:
            from ..models.classic_decoder import ClassicDecoder
            fam = CLASSIC[str(rel.config["model_type"]).lower()]
            model = ClassicDecoder(read_classic_config(rel.config), dtype=dtype, device=device)
            model.unread_keys = load_classic_state(model, rel, fam, strict=strict)
            model.generation_config = GenerationConfig.read(directory)
            model.family = fam.name
            return model
        if str(rel.config.get("model_type") or "").lower() in ("mamba", "mamba2"):
            from .recurrent import load_recurrent_state, read_recurrent_config
            model = CausalTransformer(read_recurrent_config(rel.config), dtype=dtype, device=device)
            model.unread_keys = load_recurrent_state(model, rel, strict=strict)
            model.generation_config = GenerationConfig.read(directory)
            model.family = str(rel.config["model_type"]).lower()
            return model
        fam = family_of(rel.config)
        model = CausalTransformer(read_config(rel.config), dtype=dtype, device=device)
        model.unread_keys = load_state(model, rel, fam, strict=strict)
        model.generation_config = GenerationConfig.read(directory)
        model.family = fam.name
        return model

    @staticmethod
    def save(model: CausalTransformer, directory: os.PathLike, architecture: str = "LlamaForCausalLM", family: Optional[str] = None,
             max_shard_bytes: int = 5 << 30, fp8_blocks=None, generation=None) -> None:
        from .families import FAMILIES, export_state, write_config
        from .release import save_release
        dtype = str(next(model.parameters()).dtype).replace("torch.", "")
        if family is None:
            family = next((f.name for f in FAMILIES.values() if f.architecture == architecture), None)
        if family is None:           # an architecture string outside the table: Llama naming under that label
            cfg = config_to_hf(model.config, architecture, dtype)
            save_release(to_hf_state(model, architecture), cfg, directory, max_shard_bytes, generation, fp8_blocks)
            return
        fam = FAMILIES[family]
        save_release(export_state(model, fam), write_config(model.config, family, dtype), directory, max_shard_bytes, generation, fp8_blocks)


# ------------------------------------------------------------------------------------------------ gated delta net layers
def _qkvz_from_grouped(w: torch.Tensor, hk: int, hv: int, dk: int, dv: int) -> torch.Tensor:
    """Qwen3-Next stores the fused projection grouped by key head (``[q | k | v of the group | z of the group]`` per key
    head); this library keeps ``[q of all heads | k | v | z]``."""
    rep = hv // hk
    blk = w.reshape(hk, 2 * dk + 2 * rep * dv, -1)
    q, k = blk[:, :dk], blk[:, dk:2 * dk]
    v, z = blk[:, 2 * dk:2 * dk + rep * dv], blk[:, 2 * dk + rep * dv:]
    return torch.cat([q.reshape(hk * dk, -1), k.reshape(hk * dk, -1), v.reshape(hv * dv, -1), z.reshape(hv * dv, -1)], 0)


def _ba_from_grouped(w: torch.Tensor, hk: int, hv: int) -> torch.Tensor:
    rep = hv // hk
    blk = w.reshape(hk, 2 * rep, -1)
    return torch.cat([blk[:, :rep].reshape(hv, -1), blk[:, rep:].reshape(hv, -1)], 0)


def _qkvz_to_grouped(w: torch.Tensor, hk: int, hv: int, dk: int, dv: int) -> torch.Tensor:
    rep = hv // hk
    kd, vd = hk * dk, hv * dv
    q, k, v, z = w[:kd], w[kd:2 * kd], w[2 * kd:2 * kd + vd], w[2 * kd + vd:]
    blk = torch.cat([q.reshape(hk, dk, -1), k.reshape(hk, dk, -1), v.reshape(hk, rep * dv, -1), z.reshape(hk, rep * dv, -1)], 1)
    return blk.reshape(w.shape)


def _ba_to_grouped(w: torch.Tensor, hk: int, hv: int) -> torch.Tensor:
    rep = hv // hk
    return torch.cat([w[:hv].reshape(hk, rep, -1), w[hv:].reshape(hk, rep, -1)], 1).reshape(w.shape)


def export_gated_delta_net(mixer, out: Dict[str, torch.Tensor], prefix: str = "") -> None:
    """The inverse of ``load_gated_delta_net``: a ``GatedDeltaNet`` mixer's tensors under Qwen3-Next's names and groupings."""
    out[prefix + "in_proj_qkvz.weight"] = _qkvz_to_grouped(mixer.in_proj_qkvz.weight.detach(), mixer.hk, mixer.hv, mixer.dk, mixer.dv)
    out[prefix + "in_proj_ba.weight"] = _ba_to_grouped(mixer.in_proj_ba.weight.detach(), mixer.hk, mixer.hv)
    w = mixer.conv1d.weight.detach()
    out[prefix + "conv1d.weight"] = w.reshape(w.shape[0], 1, w.shape[-1])
    out[prefix + "A_log"], out[prefix + "dt_bias"] = mixer.A_log.detach(), mixer.dt_bias.detach()
    out[prefix + "norm.weight"], out[prefix + "out_proj.weight"] = mixer.norm_weight.detach(), mixer.out_proj.weight.detach()


def load_gated_delta_net(mixer, hf: Mapping[str, torch.Tensor], prefix: str = "") -> None:
    """Copy a Qwen3-Next ``linear_attn`` layer (``in_proj_qkvz``, ``in_proj_ba``, ``conv1d``, ``A_log``, ``dt_bias``, ``norm``,
    ``out_proj``) into a ``GatedDeltaNet`` mixer, reordering the fused projections."""
    with torch.no_grad():
        mixer.in_proj_qkvz.weight.copy_(_qkvz_from_grouped(hf[prefix + "in_proj_qkvz.weight"], mixer.hk, mixer.hv, mixer.dk, mixer.dv))
        mixer.in_proj_ba.weight.copy_(_ba_from_grouped(hf[prefix + "in_proj_ba.weight"], mixer.hk, mixer.hv))
        mixer.conv1d.weight.copy_(hf[prefix + "conv1d.weight"].reshape(mixer.conv1d.weight.shape))
        mixer.A_log.copy_(hf[prefix + "A_log"])
        mixer.dt_bias.copy_(hf[prefix + "dt_bias"])
        mixer.norm_weight.copy_(hf[prefix + "norm.weight"])
        mixer.out_proj.weight.copy_(hf[prefix + "out_proj.weight"])


def load_mamba2(mixer, hf: Mapping[str, torch.Tensor], prefix: str = "") -> None:
    """Copy a transformers ``Mamba2Mixer`` (``in_proj`` as ``[z | x B C | dt]``, depthwise ``conv1d``, ``A_log``, ``D``, ``dt_bias``,
    gated ``norm``, ``out_proj``) into a ``Mamba2`` mixer: the layouts agree, only the conv weight drops its singleton axis."""
    with torch.no_grad():
        mixer.in_proj.weight.copy_(hf[prefix + "in_proj.weight"])
        mixer.out_proj.weight.copy_(hf[prefix + "out_proj.weight"])
        mixer.conv1d.weight.copy_(hf[prefix + "conv1d.weight"].reshape(mixer.conv1d.weight.shape))
        if prefix + "conv1d.bias" in hf and getattr(mixer.conv1d, "bias", None) is not None:
            mixer.conv1d.bias.copy_(hf[prefix + "conv1d.bias"])
        mixer.A_log.copy_(hf[prefix + "A_log"])
        mixer.dt_bias.copy_(hf[prefix + "dt_bias"])
        mixer.D.copy_(hf[prefix + "D"])
        mixer.norm_weight.copy_(hf[prefix + "norm.weight"])


def load_mla(mixer, hf: Mapping[str, torch.Tensor], prefix: str = "") -> None:
    """Copy a DeepSeek-V3 attention layer (``q_a_proj``, ``q_a_layernorm``, ``q_b_proj``, ``kv_a_proj_with_mqa``, ``kv_a_layernorm``,
    ``kv_b_proj``, ``o_proj``) into a ``MultiHeadLatentAttention``.  DeepSeek stores the rotary dimensions interleaved
    (pairs ``(2i, 2i + 1)``); this library rotates halves, so the rotary rows of the query up-projection (per head) and of
    the latent down-projection are reordered to ``[even | odd]``."""
    H, nope, rope = mixer.h, mixer.nope, mixer.rope
    perm = torch.cat([torch.arange(0, rope, 2), torch.arange(1, rope, 2)])
    with torch.no_grad():
        mixer.q_down.weight.copy_(hf[prefix + "q_a_proj.weight"])
        mixer.q_norm.weight.copy_(hf[prefix + "q_a_layernorm.weight"])
        qb = hf[prefix + "q_b_proj.weight"].reshape(H, nope + rope, -1).clone()
        qb[:, nope:] = qb[:, nope:][:, perm]
        mixer.q_up.weight.copy_(qb.reshape(H * (nope + rope), -1))
        kv = hf[prefix + "kv_a_proj_with_mqa.weight"].clone()
        kv[-rope:] = kv[-rope:][perm]
        mixer.kv_down.weight.copy_(kv)
        mixer.kv_norm.weight.copy_(hf[prefix + "kv_a_layernorm.weight"])
        mixer.kv_up.weight.copy_(hf[prefix + "kv_b_proj.weight"])
        mixer.o_proj.weight.copy_(hf[prefix + "o_proj.weight"])
