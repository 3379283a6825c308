"""State-space releases as ``CausalTransformer`` trees: ``MambaForCausalLM`` (selective scan, one mixer per block and no MLP) and
``Mamba2ForCausalLM`` (the SSD form with grouped B / C and a gated norm).  Every block is its mixer alone behind one norm
(``TransformerConfig(layer_types=('mamba',), layer_mlp=(False,))``); the tensors keep their layouts but for the depthwise convolution,
whose weight drops its singleton axis.  ``load_recurrent_state`` returns the release's keys nothing read; ``export_recurrent_state``
writes the same names back.

Reference: src/dew/interop/families/mamba.py, src/dew/interop/mamba2.py.
"""
from __future__ import annotations

from typing import Any, Dict, List, Mapping

import torch

from ..models.causal_transformer import CausalTransformer, TransformerConfig
from .families import _Reader, _put

RECURRENT = {"mamba": "MambaForCausalLM", "mamba2": "Mamba2ForCausalLM"}


def read_recurrent_config(cfg: Mapping[str, Any]) -> TransformerConfig:
    kind = str(cfg.get("model_type") or "").lower()
    if kind not in RECURRENT:
        raise KeyError(f"no state-space family for model_type {kind!r}; known: {sorted(RECURRENT)}")
    if cfg.get("use_bias"):
        raise NotImplementedError("biased input / output projections of a Mamba block are not built")
    if not cfg.get("use_conv_bias", True):
        raise NotImplementedError("a Mamba block whose convolution has no bias is not built")
    E = int(cfg["hidden_size"])
    common = dict(vocab_size=int(cfg["vocab_size"]), emb_features=E, num_layers=int(cfg["num_hidden_layers"]), num_heads=1, max_seq_len=int(cfg.get("max_position_embeddings", 8192)),
                  norm_eps=float(cfg.get("layer_norm_epsilon", 1e-5)), qk_norm=False, tie_embeddings=bool(cfg.get("tie_word_embeddings", kind == "mamba")),
                  layer_types=(kind,), layer_mlp=(False,))
    if kind == "mamba":
        rank = cfg.get("time_step_rank", "auto")
        options = dict(state_dim=int(cfg.get("state_size", 16)), expand=int(cfg.get("expand", 2)), conv_size=int(cfg.get("conv_kernel", 4)),
                       dt_rank=None if rank == "auto" else int(rank))
    else:
        if not cfg.get("rms_norm", True):
            raise NotImplementedError("Mamba-2 without its gated norm is not built")
        inner = int(cfg.get("expand", 2)) * E
        if int(cfg["num_heads"]) * int(cfg["head_dim"]) != inner:
            raise ValueError(f"num_heads x head_dim = {int(cfg['num_heads']) * int(cfg['head_dim'])} is not expand x hidden_size = {inner}")
        options = dict(state_dim=int(cfg.get("state_size", 128)), head_dim=int(cfg["head_dim"]), expand=int(cfg.get("expand", 2)), groups=int(cfg.get("n_groups", 1)),
                       conv_size=int(cfg.get("conv_kernel", 4)), norm_eps=float(cfg.get("layer_norm_epsilon", 1e-5)))
    return TransformerConfig(mixer_options=options, **common)


def write_recurrent_config(c: TransformerConfig, dtype: str = "bfloat16") -> Dict[str, Any]:
    kind, o = c.kinds()[0], c.mixer_options
    out = {"model_type": kind, "architectures": [RECURRENT[kind]], "vocab_size": c.vocab_size, "hidden_size": c.emb_features, "num_hidden_layers": c.num_layers,
           "layer_norm_epsilon": c.norm_eps, "tie_word_embeddings": c.tie_embeddings, "expand": o.get("expand", 2), "conv_kernel": o.get("conv_size", 4),
           "use_bias": False, "use_conv_bias": True, "torch_dtype": dtype, "dtype": dtype, "max_position_embeddings": c.max_seq_len}
    if kind == "mamba":
        out.update({"state_size": o.get("state_dim", 16), "time_step_rank": o.get("dt_rank") or "auto", "intermediate_size": o.get("expand", 2) * c.emb_features})
    else:
        inner = o.get("expand", 2) * c.emb_features
        out.update({"state_size": o.get("state_dim", 128), "head_dim": o.get("head_dim", 64), "num_heads": inner // o.get("head_dim", 64), "n_groups": o.get("groups", 1),
                    "rms_norm": True, "chunk_size": 256})
    return out


_MAMBA = ("A_log", "D", "in_proj.weight", "x_proj.weight", "dt_proj.weight", "dt_proj.bias", "out_proj.weight")
_MAMBA2 = ("A_log", "D", "dt_bias", "in_proj.weight", "out_proj.weight")


def _mixer_tensors(mixer, kind: str):
    """``(release name under 'mixer.', parameter, stored shape)`` of one block."""
    named = dict(mixer.named_parameters())
    rows = [(k, named[k], None) for k in (_MAMBA if kind == "mamba" else _MAMBA2)]
    conv = mixer.conv if kind == "mamba" else mixer.conv1d
    rows += [("conv1d.weight", conv.weight, (conv.weight.shape[0], 1, conv.weight.shape[-1])), ("conv1d.bias", conv.bias, None)]
    if kind == "mamba2":
        rows.append(("norm.weight", mixer.norm_weight, None))
    return rows


def load_recurrent_state(model: CausalTransformer, tensors: Mapping[str, torch.Tensor], strict: bool = True) -> List[str]:
    get = _Reader(tensors)
    kind = model.config.kinds()[0]
    _put(model.embed.weight, get("backbone.embeddings.weight"))
    _put(model.final_norm.weight, get("backbone.norm_f.weight"))
    if model.head is not None:
        _put(model.head.weight, get("lm_head.weight") if get.has("lm_head.weight") else get("backbone.embeddings.weight"))
    elif get.has("lm_head.weight"):
        get.read.add("lm_head.weight")
    for i, layer in enumerate(model.layers):
        pre = f"backbone.layers.{i}."
        _put(layer.input_norm.weight, get(pre + "norm.weight"))
        for name, param, _ in _mixer_tensors(layer.mixer, kind):
            _put(param, get(pre + "mixer." + name).reshape(param.shape))
    left = get.unread()
    if strict and left:
        raise KeyError(f"{len(left)} tensor(s) of the release were not read by the {kind} mapping: {left[:6]}")
    return left


def export_recurrent_state(model: CausalTransformer) -> Dict[str, torch.Tensor]:
    kind = model.config.kinds()[0]
    out = {"backbone.embeddings.weight": model.embed.weight.detach(), "backbone.norm_f.weight": model.final_norm.weight.detach()}
    if model.head is not None:
        out["lm_head.weight"] = model.head.weight.detach()
    for i, layer in enumerate(model.layers):
        pre = f"backbone.layers.{i}."
        out[pre + "norm.weight"] = layer.input_norm.weight.detach()
        for name, param, shape in _mixer_tensors(layer.mixer, kind):
            out[pre + "mixer." + name] = param.detach() if shape is None else param.detach().reshape(shape)
    return {k: v.contiguous() for k, v in out.items()}
