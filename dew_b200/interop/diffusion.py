"""Released latent-diffusion checkpoints read into this library's modules, and a pipeline assembled from a component directory.

FLUX transformer: two public layouts of the same weights -
  * the original release's (``double_blocks.N.img_attn.qkv``, ``img_mod.lin``, ``single_blocks.N.linear1`` ...), and
  * the component-directory layout (``transformer_blocks.N.attn.to_q`` / ``add_q_proj``, ``norm1.linear``, ``single_transformer_blocks.N.
    proj_mlp`` ..., where q / k / v are separate matrices and the final modulation stores (scale, shift) instead of (shift, scale)).
``flux_from_original`` / ``flux_from_components`` build a ``RectifiedFlowTransformer`` from either; ``flux_to_original`` /
``flux_to_components`` write them back (the exporters, and what the round-trip tests run against).

``autoencoder_kl_from_components`` builds an ``AutoencoderKL`` from its ``config.json`` fields and state dict (older files name the
middle attention ``query / key / value / proj_attn`` and store 1 x 1 convolutions: both are mapped).

``load_pipeline(directory)`` reads ``model_index.json``, then each component's ``config.json`` and safetensors (sharded or not):
``transformer``, ``vae``, ``text_encoder`` / ``text_encoder_2`` (CLIP, T5 through ``interop.encoders``) and the ``scheduler``'s settings.

No released checkpoint exists on this machine: the key maps are tested by round trip and by shape, not against real files.
Reference: src/dew/interop/pipeline_assembly.py, src/dew/interop/autoencoders/pretrained.py, src/dew/interop/flux.py.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch

from ..models.latent_autoencoders import AutoencoderKL
from ..models.latent_backbones import RectifiedFlowTransformer


# ------------------------------------------------------------------------------------------------ FLUX: original layout
def _orig_pairs(prefix_ours: str, prefix_theirs: str, pairs) -> List[Tuple[str, str]]:
    return [(f"{prefix_ours}{a}.{p}", f"{prefix_theirs}{b}.{p}") for a, b in pairs for p in ("weight", "bias")]


def _original_names(model: RectifiedFlowTransformer) -> List[Tuple[str, str]]:
    """(our name, the original release's name) for every parameter."""
    out = _orig_pairs("", "", [("img_in", "img_in"), ("txt_in", "txt_in"), ("time_in.fc1", "time_in.in_layer"), ("time_in.fc2", "time_in.out_layer"),
                               ("final_mod", "final_layer.adaLN_modulation.1"), ("final", "final_layer.linear")])
    if model.vector_in is not None:
        out += _orig_pairs("", "", [("vector_in.fc1", "vector_in.in_layer"), ("vector_in.fc2", "vector_in.out_layer")])
    if model.guidance_in is not None:
        out += _orig_pairs("", "", [("guidance_in.fc1", "guidance_in.in_layer"), ("guidance_in.fc2", "guidance_in.out_layer")])
    for i, blk in enumerate(model.double_blocks):
        o, t = f"double_blocks.{i}.", f"double_blocks.{i}."
        for s in ("img", "txt"):
            out += _orig_pairs(o, t, [(f"{s}_mod", f"{s}_mod.lin"), (f"{s}_qkv", f"{s}_attn.qkv")])
            out += [(f"{o}{s}_qknorm.q.weight", f"{t}{s}_attn.norm.query_norm.scale"), (f"{o}{s}_qknorm.k.weight", f"{t}{s}_attn.norm.key_norm.scale")]
            if not (s == "txt" and blk.text_pre_only):
                out += _orig_pairs(o, t, [(f"{s}_proj", f"{s}_attn.proj"), (f"{s}_fc1", f"{s}_mlp.0"), (f"{s}_fc2", f"{s}_mlp.2")])
    for i in range(len(model.single_blocks)):
        o = t = f"single_blocks.{i}."
        out += _orig_pairs(o, t, [("mod", "modulation.lin"), ("linear1", "linear1"), ("linear2", "linear2")])
        out += [(f"{o}qknorm.q.weight", f"{t}norm.query_norm.scale"), (f"{o}qknorm.k.weight", f"{t}norm.key_norm.scale")]
    own = set(model.state_dict())
    return [(a, b) for a, b in out if a in own]


def flux_to_original(model: RectifiedFlowTransformer) -> Dict[str, torch.Tensor]:
    sd = model.state_dict()
    return {theirs: sd[ours].detach().clone() for ours, theirs in _original_names(model)}


def _fill(model, mapping: Mapping[str, torch.Tensor], strict: bool) -> List[str]:
    sd = model.state_dict()
    missing = [k for k in sd if k not in mapping]
    if strict and missing:
        raise KeyError(f"the checkpoint lacks {len(missing)} tensors, e.g. {missing[:4]}")
    with torch.no_grad():
        for k, v in mapping.items():
            if k in sd:
                if tuple(sd[k].shape) != tuple(v.shape):
                    raise ValueError(f"{k}: the checkpoint holds {tuple(v.shape)}, the model {tuple(sd[k].shape)}")
                sd[k].copy_(v.to(sd[k].dtype))
    return missing


def flux_config_from_original(tensors: Mapping[str, torch.Tensor], num_heads: Optional[int] = None) -> Dict[str, Any]:
    """The model's fields read off the tensors' shapes (the original release ships no config file)."""
    d = tensors["img_in.weight"].shape[0]
    double = 1 + max(int(k.split(".")[1]) for k in tensors if k.startswith("double_blocks."))
    singles = [int(k.split(".")[1]) for k in tensors if k.startswith("single_blocks.")]
    hd = tensors["double_blocks.0.img_attn.norm.query_norm.scale"].shape[0]
    hidden = tensors["double_blocks.0.img_mlp.0.weight"].shape[0]
    return dict(patch_size=2, input_channels=tensors["img_in.weight"].shape[1] // 4, emb_features=d, num_heads=num_heads or d // hd,
                double_layers=double, single_layers=(1 + max(singles)) if singles else 0, mlp_ratio=hidden / d,
                text_features=tensors["txt_in.weight"].shape[1],
                pooled_features=tensors["vector_in.in_layer.weight"].shape[1] if "vector_in.in_layer.weight" in tensors else None,
                guidance_embed="guidance_in.in_layer.weight" in tensors)


def flux_from_original(tensors: Mapping[str, torch.Tensor], config: Optional[Mapping[str, Any]] = None, strict: bool = True, dtype=None, device=None
                       ) -> RectifiedFlowTransformer:
    cfg = dict(config) if config is not None else flux_config_from_original(tensors)
    model = RectifiedFlowTransformer(**cfg).to(device=device, dtype=dtype)
    names = dict((theirs, ours) for ours, theirs in _original_names(model))
    _fill(model, {names[k]: v for k, v in tensors.items() if k in names}, strict)
    return model


# ------------------------------------------------------------------------------------------------ FLUX: component layout
def _swap_halves(t: torch.Tensor) -> torch.Tensor:
    a, b = t.chunk(2, 0)
    return torch.cat([b, a], 0)


def flux_to_components(model: RectifiedFlowTransformer) -> Dict[str, torch.Tensor]:
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    out: Dict[str, torch.Tensor] = {}

    def put(theirs: str, ours: str, fn=lambda t: t):
        for p in ("weight", "bias"):
            if f"{ours}.{p}" in sd:
                out[f"{theirs}.{p}"] = fn(sd[f"{ours}.{p}"]).clone()
    put("x_embedder", "img_in"); put("context_embedder", "txt_in")
    put("time_text_embed.timestep_embedder.linear_1", "time_in.fc1"); put("time_text_embed.timestep_embedder.linear_2", "time_in.fc2")
    put("time_text_embed.text_embedder.linear_1", "vector_in.fc1"); put("time_text_embed.text_embedder.linear_2", "vector_in.fc2")
    put("time_text_embed.guidance_embedder.linear_1", "guidance_in.fc1"); put("time_text_embed.guidance_embedder.linear_2", "guidance_in.fc2")
    put("proj_out", "final"); put("norm_out.linear", "final_mod", _swap_halves)
    for i, blk in enumerate(model.double_blocks):
        o, t = f"double_blocks.{i}.", f"transformer_blocks.{i}."
        put(t + "norm1.linear", o + "img_mod"); put(t + "norm1_context.linear", o + "txt_mod")
        for part, (tq, tk, tv) in (("img", ("attn.to_q", "attn.to_k", "attn.to_v")), ("txt", ("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj"))):
            for j, name in enumerate((tq, tk, tv)):
                put(t + name, o + f"{part}_qkv", lambda x, j=j: x.chunk(3, 0)[j])
        out[t + "attn.norm_q.weight"], out[t + "attn.norm_k.weight"] = sd[o + "img_qknorm.q.weight"].clone(), sd[o + "img_qknorm.k.weight"].clone()
        out[t + "attn.norm_added_q.weight"], out[t + "attn.norm_added_k.weight"] = sd[o + "txt_qknorm.q.weight"].clone(), sd[o + "txt_qknorm.k.weight"].clone()
        put(t + "attn.to_out.0", o + "img_proj"); put(t + "ff.net.0.proj", o + "img_fc1"); put(t + "ff.net.2", o + "img_fc2")
        if not blk.text_pre_only:
            put(t + "attn.to_add_out", o + "txt_proj"); put(t + "ff_context.net.0.proj", o + "txt_fc1"); put(t + "ff_context.net.2", o + "txt_fc2")
    for i, blk in enumerate(model.single_blocks):
        o, t = f"single_blocks.{i}.", f"single_transformer_blocks.{i}."
        d = blk.linear2.weight.shape[0]
        put(t + "norm.linear", o + "mod")
        for j, name in enumerate(("attn.to_q", "attn.to_k", "attn.to_v")):
            put(t + name, o + "linear1", lambda x, j=j: x[j * d:(j + 1) * d])
        put(t + "proj_mlp", o + "linear1", lambda x: x[3 * d:])
        out[t + "attn.norm_q.weight"], out[t + "attn.norm_k.weight"] = sd[o + "qknorm.q.weight"].clone(), sd[o + "qknorm.k.weight"].clone()
        put(t + "proj_out", o + "linear2")
    return out


def flux_config_from_components(config: Mapping[str, Any]) -> Dict[str, Any]:
    heads, hd = int(config["num_attention_heads"]), int(config["attention_head_dim"])
    return dict(patch_size=int(config.get("patch_size", 1)) * 2, input_channels=int(config["in_channels"]) // 4, emb_features=heads * hd, num_heads=heads,
                double_layers=int(config["num_layers"]), single_layers=int(config["num_single_layers"]), text_features=int(config["joint_attention_dim"]),
                pooled_features=config.get("pooled_projection_dim"), guidance_embed=bool(config.get("guidance_embeds", False)),
                axes_dims=tuple(config["axes_dims_rope"]) if config.get("axes_dims_rope") else None)


def flux_from_components(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], strict: bool = True, dtype=None, device=None
                         ) -> RectifiedFlowTransformer:
    model = RectifiedFlowTransformer(**flux_config_from_components(config)).to(device=device, dtype=dtype)
    mapping: Dict[str, torch.Tensor] = {}

    def take(ours: str, theirs: str, fn=lambda t: t):
        for p in ("weight", "bias"):
            if f"{theirs}.{p}" in tensors:
                mapping[f"{ours}.{p}"] = fn(tensors[f"{theirs}.{p}"])

    def fuse(ours: str, names, p_list=("weight", "bias")):
        for p in p_list:
            if all(f"{n}.{p}" in tensors for n in names):
                mapping[f"{ours}.{p}"] = torch.cat([tensors[f"{n}.{p}"] for n in names], 0)
    take("img_in", "x_embedder"); take("txt_in", "context_embedder")
    take("time_in.fc1", "time_text_embed.timestep_embedder.linear_1"); take("time_in.fc2", "time_text_embed.timestep_embedder.linear_2")
    take("vector_in.fc1", "time_text_embed.text_embedder.linear_1"); take("vector_in.fc2", "time_text_embed.text_embedder.linear_2")
    take("guidance_in.fc1", "time_text_embed.guidance_embedder.linear_1"); take("guidance_in.fc2", "time_text_embed.guidance_embedder.linear_2")
    take("final", "proj_out"); take("final_mod", "norm_out.linear", _swap_halves)
    for i, blk in enumerate(model.double_blocks):
        o, t = f"double_blocks.{i}.", f"transformer_blocks.{i}."
        take(o + "img_mod", t + "norm1.linear"); take(o + "txt_mod", t + "norm1_context.linear")
        fuse(o + "img_qkv", [t + "attn.to_q", t + "attn.to_k", t + "attn.to_v"])
        fuse(o + "txt_qkv", [t + "attn.add_q_proj", t + "attn.add_k_proj", t + "attn.add_v_proj"])
        for ours, theirs in (("img_qknorm.q", "attn.norm_q"), ("img_qknorm.k", "attn.norm_k"), ("txt_qknorm.q", "attn.norm_added_q"), ("txt_qknorm.k", "attn.norm_added_k")):
            if t + theirs + ".weight" in tensors:
                mapping[o + ours + ".weight"] = tensors[t + theirs + ".weight"]
        take(o + "img_proj", t + "attn.to_out.0"); take(o + "img_fc1", t + "ff.net.0.proj"); take(o + "img_fc2", t + "ff.net.2")
        take(o + "txt_proj", t + "attn.to_add_out"); take(o + "txt_fc1", t + "ff_context.net.0.proj"); take(o + "txt_fc2", t + "ff_context.net.2")
    for i in range(len(model.single_blocks)):
        o, t = f"single_blocks.{i}.", f"single_transformer_blocks.{i}."
        take(o + "mod", t + "norm.linear")
        fuse(o + "linear1", [t + "attn.to_q", t + "attn.to_k", t + "attn.to_v", t + "proj_mlp"])
        for ours, theirs in (("qknorm.q", "attn.norm_q"), ("qknorm.k", "attn.norm_k")):
            if t + theirs + ".weight" in tensors:
                mapping[o + ours + ".weight"] = tensors[t + theirs + ".weight"]
        take(o + "linear2", t + "proj_out")
    _fill(model, mapping, strict)
    return model


# ------------------------------------------------------------------------------------------------ AutoencoderKL
_LEGACY_ATTENTION = {"query": "to_q", "key": "to_k", "value": "to_v", "proj_attn": "to_out.0"}


def autoencoder_kl_from_components(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], strict: bool = True, dtype=None, device=None
                                   ) -> AutoencoderKL:
    model = AutoencoderKL(in_channels=int(config.get("in_channels", 3)), latent_channels=int(config.get("latent_channels", 4)),
                          block_out_channels=tuple(config.get("block_out_channels", (128, 256, 512, 512))),
                          layers_per_block=int(config.get("layers_per_block", 2)), norm_groups=int(config.get("norm_num_groups", 32)),
                          scaling_factor=float(config.get("scaling_factor", 0.18215)), shift_factor=config.get("shift_factor"),
                          use_quant_conv=bool(config.get("use_quant_conv", True)), mid_attention=bool(config.get("mid_block_add_attention", True))
                          ).to(device=device, dtype=dtype)
    own = model.state_dict()
    mapping: Dict[str, torch.Tensor] = {}
    for k, v in tensors.items():
        parts = k.split(".")
        if "attentions" in parts:
            at = parts.index("attentions") + 2
            if parts[at] in _LEGACY_ATTENTION:
                parts[at:at + 1] = _LEGACY_ATTENTION[parts[at]].split(".")
                k = ".".join(parts)
            if k in own and v.dim() == 4 and own[k].dim() == 2:             # 1 x 1 convolutions of the first releases
                v = v[:, :, 0, 0]
        mapping[k] = v
    _fill(model, mapping, strict)
    return model


# ------------------------------------------------------------------------------------------------ a pipeline from a directory
def _read_tensors(folder: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    index = [f for f in os.listdir(folder) if f.endswith(".safetensors.index.json")]
    if index:
        with open(os.path.join(folder, index[0])) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = sorted(f for f in os.listdir(folder) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors file in {folder}")
    out: Dict[str, torch.Tensor] = {}
    for name in files:
        out.update(load_file(os.path.join(folder, name)))
    return out


@dataclass
class Pipeline:
    kind: str
    transformer: Optional[torch.nn.Module] = None
    vae: Optional[torch.nn.Module] = None
    text_encoders: Dict[str, torch.nn.Module] = field(default_factory=dict)
    scheduler: Dict[str, Any] = field(default_factory=dict)
    unread: Dict[str, List[str]] = field(default_factory=dict)             # component -> parameters the files did not hold

    def solver_settings(self) -> Dict[str, Any]:
        """What a sampler needs of the scheduler's record: the flow-matching time shift (fixed, or resolution-dependent between
        ``base_shift`` and ``max_shift``) and the number of training timesteps."""
        s = self.scheduler
        return {"shift": s.get("shift", 1.0), "dynamic": bool(s.get("use_dynamic_shifting", False)), "base_shift": s.get("base_shift", 0.5),
                "max_shift": s.get("max_shift", 1.15), "base_tokens": s.get("base_image_seq_len", 256), "max_tokens": s.get("max_image_seq_len", 4096),
                "train_timesteps": s.get("num_train_timesteps", 1000)}


def load_pipeline(directory: str, components: Optional[List[str]] = None, strict: bool = True, dtype=None, device=None) -> Pipeline:
    with open(os.path.join(directory, "model_index.json")) as f:
        index = json.load(f)
    pipe = Pipeline(kind=index.get("_class_name", ""))
    from . import encoders as E
    for name, spec in index.items():
        if name.startswith("_") or not isinstance(spec, list) or spec[0] is None:
            continue
        if components is not None and name not in components:
            continue
        folder = os.path.join(directory, name)
        cls = spec[1]
        cfg_file = next((os.path.join(folder, f) for f in ("config.json", "scheduler_config.json") if os.path.exists(os.path.join(folder, f))), None)
        config = json.load(open(cfg_file)) if cfg_file else {}
        if name == "scheduler":
            pipe.scheduler = config
        elif cls == "AutoencoderKL":
            pipe.vae = autoencoder_kl_from_components(config, _read_tensors(folder), strict, dtype, device)
        elif cls == "FluxTransformer2DModel":
            pipe.transformer = flux_from_components(config, _read_tensors(folder), strict, dtype, device)
        elif cls in ("CLIPTextModel", "CLIPTextModelWithProjection"):
            pipe.text_encoders[name], pipe.unread[name] = E.clip_text(config, _read_tensors(folder), dtype, device)
        elif cls == "T5EncoderModel":
            pipe.text_encoders[name], pipe.unread[name] = E.t5_encoder(config, _read_tensors(folder), dtype, device)
        elif name in ("tokenizer", "tokenizer_2", "feature_extractor", "image_encoder", "safety_checker"):
            continue
        else:
            raise ValueError(f"component {name!r} is a {cls}, which this loader does not build (known: AutoencoderKL, FluxTransformer2DModel, "
                             "CLIPTextModel, T5EncoderModel, a scheduler)")
    return pipe
