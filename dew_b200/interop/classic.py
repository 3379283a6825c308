"""Published checkpoints of the decoder lineage before RMSNorm and gated MLPs, read into (and written from) ``ClassicDecoder``: GPT-2
(Conv1D weights stored ``[in, out]``, learned positions), GPTBigCode (multi-query GPT-2 with Linear weights), GPT-NeoX (two-norm parallel
block, q | k | v interleaved per head, a quarter of each head rotating), Falcon (7B: one-norm parallel block, multi-query; 40B / 180B: grouped keys stored per group, one or two norms), GPT-J (one-norm
parallel block, rotary pairs over part of each head, a biased head), Phi
(one-norm parallel block, half of each head rotating, a biased output head), OPT (position table offset by two, ReLU, pre- or post-norm, the
350m size's embedding projections), BLOOM (ALiBi, a norm on the embeddings, per-head q | k | v) and StarCoder2 (rotary, grouped keys, a
sliding window).  One ``ClassicFamily`` row per family says how its ``config.json`` reads as a ``ClassicConfig`` and under which names and
storage forms its tensors sit; ``load_state`` returns the keys nothing read, so a partial load cannot pass silently, and
``export_state`` writes the same names back.

Reference: src/dew/interop/families/gpt2.py, gpt_bigcode.py, (GPT-J: the parts of decoder_parts.py), gpt_neox.py, falcon.py, phi.py, opt.py, bloom.py, starcoder2.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional

import torch

from ..models.classic_decoder import ClassicConfig, ClassicDecoder
from .families import _Reader, _put, head_order

_ACT = {"gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu_fast": "gelu_tanh", "gelu": "gelu", "relu": "relu", "silu": "silu"}


def _theta(cfg) -> float:
    return float((cfg.get("rope_parameters") or {}).get("rope_theta", cfg.get("rope_theta", 10000.0)))


def _fraction(cfg, default: float) -> float:
    rope = cfg.get("rope_parameters") or {}
    return float(rope.get("partial_rotary_factor", cfg.get("partial_rotary_factor", cfg.get("rotary_pct", default))))


def _gpt2(cfg):
    return dict(vocab_size=cfg["vocab_size"], emb_features=cfg["n_embd"], num_layers=cfg["n_layer"], num_heads=cfg["n_head"],
                mlp_features=cfg.get("n_inner") or 4 * cfg["n_embd"], max_seq_len=cfg["n_positions"], norm_eps=cfg.get("layer_norm_epsilon", 1e-5),
                activation=_ACT[cfg.get("activation_function", "gelu_new")], tie_embeddings=bool(cfg.get("tie_word_embeddings", True)))


def _gpt_bigcode(cfg):
    return dict(_gpt2(cfg), num_kv_heads=1 if cfg.get("multi_query", True) else None)


def _gpt_neox(cfg):
    return dict(vocab_size=cfg["vocab_size"], emb_features=cfg["hidden_size"], num_layers=cfg["num_hidden_layers"], num_heads=cfg["num_attention_heads"],
                mlp_features=cfg["intermediate_size"], max_seq_len=cfg["max_position_embeddings"], norm_eps=cfg.get("layer_norm_eps", 1e-5),
                activation=_ACT[cfg.get("hidden_act", "gelu")], positions="rotary", rope_theta=_theta(cfg), rotary_fraction=_fraction(cfg, 0.25),
                block="parallel" if cfg.get("use_parallel_residual", True) else "sequential", parallel_norms=2,
                attn_bias=bool(cfg.get("attention_bias", True)), tie_embeddings=bool(cfg.get("tie_word_embeddings", False)))


def _gptj(cfg):
    E, H = cfg["n_embd"], cfg["n_head"]
    return dict(vocab_size=cfg["vocab_size"], emb_features=E, num_layers=cfg["n_layer"], num_heads=H, mlp_features=cfg.get("n_inner") or 4 * E,
                max_seq_len=cfg["n_positions"], norm_eps=cfg.get("layer_norm_epsilon", 1e-5), activation=_ACT[cfg.get("activation_function", "gelu_new")],
                positions="rotary", rope_theta=_theta(cfg), rotary_fraction=float(cfg.get("rotary_dim") or E // H) / (E // H), block="parallel",
                parallel_norms=1, attn_bias=False, mlp_bias=True, tie_embeddings=bool(cfg.get("tie_word_embeddings", False)), head_bias=True)


def _falcon(cfg):
    new = bool(cfg.get("new_decoder_architecture"))
    if cfg.get("alibi") or not (new or cfg.get("parallel_attn", True)):
        raise NotImplementedError("of Falcon, the rotary parallel-block layouts are built: 7B's (one norm, multi-query) and 40B / 180B's (grouped keys, "
                                  "one or two norms) - not ALiBi, nor the sequential block")
    E = cfg["hidden_size"]
    kv = int(cfg.get("num_kv_heads") or cfg["num_attention_heads"]) if new else (1 if cfg.get("multi_query", True) else None)
    norms = int(cfg.get("num_ln_in_parallel_attn") or 2) if new else 1
    return dict(vocab_size=cfg["vocab_size"], emb_features=E, num_layers=cfg["num_hidden_layers"], num_heads=cfg["num_attention_heads"],
                num_kv_heads=kv, parallel_norms=norms, mlp_features=cfg.get("ffn_hidden_size") or 4 * E,
                max_seq_len=cfg.get("max_position_embeddings", 2048), norm_eps=cfg.get("layer_norm_epsilon", 1e-5), activation=_ACT[cfg.get("activation", "gelu")],
                positions="rotary", rope_theta=_theta(cfg), block="parallel", attn_bias=bool(cfg.get("bias", False)),
                mlp_bias=bool(cfg.get("bias", False)), tie_embeddings=bool(cfg.get("tie_word_embeddings", True)))


def _phi(cfg):
    if cfg.get("qk_layernorm"):
        raise NotImplementedError("Phi with q / k LayerNorms is not built")
    return dict(vocab_size=cfg["vocab_size"], emb_features=cfg["hidden_size"], num_layers=cfg["num_hidden_layers"], num_heads=cfg["num_attention_heads"],
                num_kv_heads=cfg.get("num_key_value_heads"), mlp_features=cfg["intermediate_size"], max_seq_len=cfg["max_position_embeddings"],
                norm_eps=cfg.get("layer_norm_eps", 1e-5), activation=_ACT[cfg.get("hidden_act", "gelu_new")], positions="rotary", rope_theta=_theta(cfg),
                rotary_fraction=_fraction(cfg, 0.5), block="parallel", parallel_norms=1, tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
                head_bias=True)


def _opt(cfg):
    before = bool(cfg.get("do_layer_norm_before", True))
    E, Ew = cfg["hidden_size"], cfg.get("word_embed_proj_dim") or cfg["hidden_size"]
    return dict(vocab_size=cfg["vocab_size"], emb_features=E, num_layers=cfg["num_hidden_layers"], num_heads=cfg["num_attention_heads"],
                mlp_features=cfg["ffn_dim"], max_seq_len=cfg["max_position_embeddings"], position_offset=2, activation=_ACT[cfg.get("activation_function", "relu")],
                block="sequential" if before else "post_norm", final_norm=before and not cfg.get("_remove_final_layer_norm", False),
                attn_bias=bool(cfg.get("enable_bias", True)), mlp_bias=bool(cfg.get("enable_bias", True)), embed_proj=Ew if Ew != E else None,
                tie_embeddings=bool(cfg.get("tie_word_embeddings", True)))


def _bloom(cfg):
    if cfg.get("apply_residual_connection_post_layernorm"):
        raise NotImplementedError("BLOOM with the residual taken after the norm is not built")
    E = cfg["hidden_size"]
    return dict(vocab_size=cfg["vocab_size"], emb_features=E, num_layers=cfg["n_layer"], num_heads=cfg["n_head"], mlp_features=4 * E,
                max_seq_len=cfg.get("seq_length", 2048), norm_eps=cfg.get("layer_norm_epsilon", 1e-5), activation="gelu_tanh", positions="alibi",
                embed_norm=True, tie_embeddings=bool(cfg.get("tie_word_embeddings", True)))


def _starcoder2(cfg):
    return dict(vocab_size=cfg["vocab_size"], emb_features=cfg["hidden_size"], num_layers=cfg["num_hidden_layers"], num_heads=cfg["num_attention_heads"],
                num_kv_heads=cfg.get("num_key_value_heads"), mlp_features=cfg["intermediate_size"], max_seq_len=cfg["max_position_embeddings"],
                norm_eps=cfg.get("norm_epsilon", 1e-5), activation=_ACT[cfg.get("hidden_act", "gelu_pytorch_tanh")], positions="rotary", rope_theta=_theta(cfg),
                attn_bias=bool(cfg.get("use_bias", True)), mlp_bias=bool(cfg.get("use_bias", True)), window=cfg.get("sliding_window"),
                tie_embeddings=bool(cfg.get("tie_word_embeddings", True)))


@dataclass(frozen=True)
class ClassicFamily:
    name: str
    architecture: str
    read_config: Callable[[Mapping[str, Any]], Dict[str, Any]]
    names: Mapping[str, str]                       # slot -> the release's name; layer slots are formatted with the layer index
    qkv: str = "split"                             # split: q, k, v tensors | packed: one tensor q | k | v | by_head: one tensor, (q, k, v) per head
                                                   # | grouped: one tensor, per key head its queries then its key then its value
    rotary_pairs: bool = False                     # the release rotates pairs (2i, 2i + 1) of a head's rotating part, not its halves
    transposed: bool = False                       # GPT-2's Conv1D stores weights [in, out]
    extra_config: Mapping[str, Any] = field(default_factory=dict)


def _names(stem: str, layer: str, **slots) -> Dict[str, str]:
    return {k: (stem + layer + v[1:] if v.startswith("@") else stem + v if not v.startswith("/") else v[1:]) for k, v in slots.items()}


CLASSIC: Dict[str, ClassicFamily] = {f.name: f for f in (
    ClassicFamily("gpt2", "GPT2LMHeadModel", _gpt2, _names(
        "transformer.", "h.{}.", embed="wte", positions="wpe", final_norm="ln_f", head="/lm_head", norm1="@ln_1", norm2="@ln_2", qkv="@attn.c_attn",
        out="@attn.c_proj", fc1="@mlp.c_fc", fc2="@mlp.c_proj"), qkv="packed", transposed=True),
    ClassicFamily("gpt_bigcode", "GPTBigCodeForCausalLM", _gpt_bigcode, _names(
        "transformer.", "h.{}.", embed="wte", positions="wpe", final_norm="ln_f", head="/lm_head", norm1="@ln_1", norm2="@ln_2", qkv="@attn.c_attn",
        out="@attn.c_proj", fc1="@mlp.c_fc", fc2="@mlp.c_proj"), qkv="packed"),
    ClassicFamily("gpt_neox", "GPTNeoXForCausalLM", _gpt_neox, _names(
        "gpt_neox.", "layers.{}.", embed="embed_in", final_norm="final_layer_norm", head="/embed_out", norm1="@input_layernorm", norm2="@post_attention_layernorm",
        qkv="@attention.query_key_value", out="@attention.dense", fc1="@mlp.dense_h_to_4h", fc2="@mlp.dense_4h_to_h"), qkv="by_head"),
    ClassicFamily("falcon", "FalconForCausalLM", _falcon, _names(
        "transformer.", "h.{}.", embed="word_embeddings", final_norm="ln_f", head="/lm_head", norm1="@input_layernorm", qkv="@self_attention.query_key_value",
        out="@self_attention.dense", fc1="@mlp.dense_h_to_4h", fc2="@mlp.dense_4h_to_h"), qkv="packed"),
    ClassicFamily("falcon_grouped", "FalconForCausalLM", _falcon, _names(
        "transformer.", "h.{}.", embed="word_embeddings", final_norm="ln_f", head="/lm_head", norm1="@ln_attn", norm2="@ln_mlp", qkv="@self_attention.query_key_value",
        out="@self_attention.dense", fc1="@mlp.dense_h_to_4h", fc2="@mlp.dense_4h_to_h"), qkv="grouped"),
    ClassicFamily("falcon_grouped_one_norm", "FalconForCausalLM", _falcon, _names(
        "transformer.", "h.{}.", embed="word_embeddings", final_norm="ln_f", head="/lm_head", norm1="@input_layernorm", qkv="@self_attention.query_key_value",
        out="@self_attention.dense", fc1="@mlp.dense_h_to_4h", fc2="@mlp.dense_4h_to_h"), qkv="grouped"),
    ClassicFamily("gptj", "GPTJForCausalLM", _gptj, _names(
        "transformer.", "h.{}.", embed="wte", final_norm="ln_f", head="/lm_head", norm1="@ln_1", q="@attn.q_proj", k="@attn.k_proj", v="@attn.v_proj",
        out="@attn.out_proj", fc1="@mlp.fc_in", fc2="@mlp.fc_out"), rotary_pairs=True),
    ClassicFamily("phi", "PhiForCausalLM", _phi, _names(
        "model.", "layers.{}.", embed="embed_tokens", final_norm="final_layernorm", head="/lm_head", norm1="@input_layernorm", q="@self_attn.q_proj",
        k="@self_attn.k_proj", v="@self_attn.v_proj", out="@self_attn.dense", fc1="@mlp.fc1", fc2="@mlp.fc2")),
    ClassicFamily("opt", "OPTForCausalLM", _opt, _names(
        "model.decoder.", "layers.{}.", embed="embed_tokens", positions="embed_positions", final_norm="final_layer_norm", head="/lm_head",
        project_in="project_in", project_out="project_out", norm1="@self_attn_layer_norm", norm2="@final_layer_norm", q="@self_attn.q_proj",
        k="@self_attn.k_proj", v="@self_attn.v_proj", out="@self_attn.out_proj", fc1="@fc1", fc2="@fc2")),
    ClassicFamily("bloom", "BloomForCausalLM", _bloom, _names(
        "transformer.", "h.{}.", embed="word_embeddings", embed_norm="word_embeddings_layernorm", final_norm="ln_f", head="/lm_head", norm1="@input_layernorm",
        norm2="@post_attention_layernorm", qkv="@self_attention.query_key_value", out="@self_attention.dense", fc1="@mlp.dense_h_to_4h",
        fc2="@mlp.dense_4h_to_h"), qkv="by_head"),
    ClassicFamily("starcoder2", "Starcoder2ForCausalLM", _starcoder2, _names(
        "model.", "layers.{}.", embed="embed_tokens", final_norm="norm", head="/lm_head", norm1="@input_layernorm", norm2="@post_attention_layernorm",
        q="@self_attn.q_proj", k="@self_attn.k_proj", v="@self_attn.v_proj", out="@self_attn.o_proj", fc1="@mlp.c_fc", fc2="@mlp.c_proj")),
)}


def classic_family_of(cfg: Mapping[str, Any]) -> ClassicFamily:
    mt = str(cfg.get("model_type") or "").lower()
    if mt == "falcon" and cfg.get("new_decoder_architecture"):
        return CLASSIC["falcon_grouped" if int(cfg.get("num_ln_in_parallel_attn") or 2) == 2 else "falcon_grouped_one_norm"]
    if mt in CLASSIC:
        return CLASSIC[mt]
    arch = (cfg.get("architectures") or [""])[0]
    for fam in CLASSIC.values():
        if fam.architecture == arch:
            return fam
    raise KeyError(f"no classic decoder family for model_type {mt!r} / architectures {cfg.get('architectures')}; known: {sorted(CLASSIC)}")


def read_classic_config(cfg: Mapping[str, Any]) -> ClassicConfig:
    return ClassicConfig(**classic_family_of(cfg).read_config(cfg))


# ------------------------------------------------------------------------------------------------ tensors
def _qkv_to_ours(t: torch.Tensor, fam: ClassicFamily, H: int, Hkv: int, D: int, order: Optional[torch.Tensor]) -> torch.Tensor:
    """A release's fused q | k | v weight ``[rows, in]`` or bias ``[rows]`` as this library packs it: all query heads, all key heads, all
    value heads, with every q and k head's dimensions in rotary layout order."""
    if fam.qkv == "by_head":
        per = t.reshape(H, 3, D, -1)
        t = torch.cat([per[:, 0], per[:, 1], per[:, 2]], 0).reshape(t.shape)
    elif fam.qkv == "grouped":
        per = t.reshape(Hkv, H // Hkv + 2, D, -1)
        t = torch.cat([per[:, :-2].reshape(H, D, -1), per[:, -2], per[:, -1]], 0).reshape(t.shape)
    if order is not None:
        heads = t.reshape(H + 2 * Hkv, D, -1).clone()
        heads[: H + Hkv] = heads[: H + Hkv][:, order]
        t = heads.reshape(t.shape)
    return t


def _qkv_to_theirs(t: torch.Tensor, fam: ClassicFamily, H: int, Hkv: int, D: int, order: Optional[torch.Tensor]) -> torch.Tensor:
    if order is not None:
        heads = t.reshape(H + 2 * Hkv, D, -1).clone()
        heads[: H + Hkv] = heads[: H + Hkv][:, torch.argsort(order)]
        t = heads.reshape(t.shape)
    if fam.qkv == "by_head":
        parts = t.reshape(3, H, D, -1)
        t = torch.stack([parts[0], parts[1], parts[2]], 1).reshape(t.shape)
    elif fam.qkv == "grouped":
        heads = t.reshape(H + 2 * Hkv, D, -1)
        q, k, v = heads[:H].reshape(Hkv, H // Hkv, D, -1), heads[H:H + Hkv, None], heads[H + Hkv:, None]
        t = torch.cat([q, k, v], 1).reshape(t.shape)
    return t


def _slots(model: ClassicDecoder):
    """``(slot, module)`` for everything outside the layers that the model has."""
    return [(s, m) for s, m in (("embed", model.embed), ("positions", model.positions), ("embed_norm", model.embed_norm), ("final_norm", model.final_norm),
                                ("project_in", model.project_in), ("project_out", model.project_out), ("head", model.head)) if m is not None]


def load_classic_state(model: ClassicDecoder, tensors: Mapping[str, torch.Tensor], family: ClassicFamily, strict: bool = True) -> List[str]:
    get = _Reader(tensors)
    c = model.config
    H, Hkv, D = c.num_heads, c.num_kv_heads or c.num_heads, c.head_dim
    order = head_order(D, int(D * c.rotary_fraction), family.rotary_pairs) if c.positions == "rotary" else None
    if family.qkv == "by_head" and Hkv != H:
        raise ValueError("per-head interleaved q | k | v storage holds as many key heads as query heads")

    def weight(key):
        w = get(key + ".weight")
        return w.t() if family.transposed and w.dim() == 2 else w

    def module(m, key, matrix=True):
        _put(m.weight, weight(key) if matrix else get(key + ".weight"))
        if getattr(m, "bias", None) is not None:
            _put(m.bias, get(key + ".bias"))
    for slot, m in _slots(model):
        key = family.names[slot]
        if slot == "head" and not get.has(key + ".weight"):
            raise KeyError(f"the model has an output head of its own and the release holds none under {key}")
        module(m, key, matrix=False)
    if model.head is None and get.has(family.names["head"] + ".weight"):
        get.read.add(family.names["head"] + ".weight")                # a tied release may still store the copy
    for i, layer in enumerate(model.layers):
        n = {k: v.format(i) for k, v in family.names.items()}
        module(layer.norm1, n["norm1"], matrix=False)
        if layer.norm2 is not None:
            module(layer.norm2, n["norm2"], matrix=False)
        if family.qkv == "split":
            w = torch.cat([weight(n[s]) for s in "qkv"], 0)
            b = torch.cat([get(n[s] + ".bias") for s in "qkv"], 0) if layer.qkv.bias is not None else None
        else:
            w = weight(n["qkv"])
            b = get(n["qkv"] + ".bias") if layer.qkv.bias is not None else None
        _put(layer.qkv.weight, _qkv_to_ours(w, family, H, Hkv, D, order))
        if b is not None:
            _put(layer.qkv.bias, _qkv_to_ours(b, family, H, Hkv, D, order))
        for slot in ("out", "fc1", "fc2"):
            module(getattr(layer, slot), n[slot])
    left = [k for k in get.unread() if not k.endswith((".attn.bias", ".attn.masked_bias", ".attention.bias", ".attention.masked_bias"))]   # causal-mask buffers
    if strict and left:
        raise KeyError(f"{len(left)} tensor(s) of the release were not read by the {family.name} mapping: {left[:6]}")
    return left


def export_classic_state(model: ClassicDecoder, family: ClassicFamily) -> Dict[str, torch.Tensor]:
    c = model.config
    H, Hkv, D = c.num_heads, c.num_kv_heads or c.num_heads, c.head_dim
    order = head_order(D, int(D * c.rotary_fraction), family.rotary_pairs) if c.positions == "rotary" else None
    out: Dict[str, torch.Tensor] = {}

    def module(m, key, matrix=True):
        w = m.weight.detach()
        out[key + ".weight"] = w.t() if family.transposed and matrix and w.dim() == 2 else w
        if getattr(m, "bias", None) is not None:
            out[key + ".bias"] = m.bias.detach()
    for slot, m in _slots(model):
        module(m, family.names[slot], matrix=False)
    for i, layer in enumerate(model.layers):
        n = {k: v.format(i) for k, v in family.names.items()}
        module(layer.norm1, n["norm1"], matrix=False)
        if layer.norm2 is not None:
            module(layer.norm2, n["norm2"], matrix=False)
        w = _qkv_to_theirs(layer.qkv.weight.detach(), family, H, Hkv, D, order)
        b = None if layer.qkv.bias is None else _qkv_to_theirs(layer.qkv.bias.detach(), family, H, Hkv, D, order)
        if family.qkv == "split":
            cuts = (0, H * D, (H + Hkv) * D, (H + 2 * Hkv) * D)
            for j, s in enumerate("qkv"):
                out[n[s] + ".weight"] = w[cuts[j]:cuts[j + 1]]
                if b is not None:
                    out[n[s] + ".bias"] = b[cuts[j]:cuts[j + 1]]
        else:
            out[n["qkv"] + ".weight"] = w.t() if family.transposed else w
            if b is not None:
                out[n["qkv"] + ".bias"] = b
        for slot in ("out", "fc1", "fc2"):
            module(getattr(layer, slot), n[slot])
    return {k: v.contiguous() for k, v in out.items()}


def load_classic(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], dtype=None, device=None) -> ClassicDecoder:
    """A ``ClassicDecoder`` built from a release's ``config.json`` mapping and its tensors."""
    fam = classic_family_of(config)
    model = ClassicDecoder(ClassicConfig(**fam.read_config(config)), dtype=dtype, device=device)
    load_classic_state(model, tensors, fam)
    return model
