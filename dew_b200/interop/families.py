"""Decoder families as their releases store them: one ``Family`` per published architecture says how its ``config.json``
reads as a ``TransformerConfig`` and where its tensors differ from the Llama naming (fused projections, biases, norm
offsets, extra norms, expert naming).  ``family_of(config)`` picks the entry by ``model_type`` / ``architectures``;
``load_state`` / ``export_state`` move tensors between a release's names and a ``CausalTransformer``, and ``load_state``
returns the release's keys nothing read, so a silent partial load cannot happen.

Families: llama, mistral, qwen2 (q/k/v bias), dream (qwen2's tensors under bidirectional attention), qwen3 (per-head q/k norm), qwen3_moe, qwen2_moe (a gated shared expert), mixtral, gemma (norm weight stored
minus one, GeGLU, scaled embeddings), gemma2 (output norms on every sub-layer, soft-capped logits, alternating local /
global layers, query scale), phi3 (fused qkv and gate_up on disk), granite (embedding / attention / residual multipliers, logits scaling), olmo2 (no pre-norms: every sub-layer's output is
normalised instead; q and k normalised over all heads at once), olmo3 (olmo2 with sliding layers on an unscaled rotary table), gemma3 (gemma2's
block with per-head q/k norms and one rotary base per layer kind), smollm3 (every fourth layer attends without positions), glm4 (half of every head rotates, as pairs; output norms; fused gate_up), qwen3_next (gated delta-rule layers with every fourth a gated softmax attention layer, a quarter of each head rotating, zero-centred norms,
routed experts beside a gated shared expert), gpt_oss (attention sinks and biases, sliding / full layers, a router over the top logits, biased clamped-GLU experts stored interleaved), deepseek_v3 (latent attention stored with
interleaved rotary pairs, dense layers first, then sigmoid-routed experts in groups with a selection bias beside shared experts).

Reference: src/dew/interop/decoder_families.py, decoder_config.py, decoder_parts.py (family tables), unread.py (keys
nothing read), hf_decoders.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import math

import torch

from ..models.causal_transformer import CausalTransformer, Mixture, TransformerConfig


def _rope(cfg: Mapping[str, Any]) -> Tuple[float, Optional[dict]]:
    rope = cfg.get("rope_parameters") or {}
    theta = rope.get("rope_theta", cfg.get("rope_theta", 10000.0))
    scaling = cfg.get("rope_scaling")
    if scaling is None and rope.get("rope_type", "default") != "default":
        scaling = {k: v for k, v in rope.items() if k != "rope_theta"}
    return float(theta), scaling


def _common(cfg: Mapping[str, Any], **over) -> Dict[str, Any]:
    heads = cfg["num_attention_heads"]
    theta, scaling = _rope(cfg)
    out = dict(vocab_size=cfg["vocab_size"], emb_features=cfg["hidden_size"], num_layers=cfg["num_hidden_layers"], num_heads=heads,
               num_kv_heads=cfg.get("num_key_value_heads") or heads, head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
               mlp_features=cfg["intermediate_size"], max_seq_len=cfg.get("max_position_embeddings", 4096), rope_theta=theta,
               rope_scaling=scaling, norm_eps=cfg.get("rms_norm_eps", 1e-6), qk_norm=False,
               tie_embeddings=bool(cfg.get("tie_word_embeddings", False)))
    out.update(over)
    return out


def _mixture(cfg: Mapping[str, Any], always_norm: bool) -> Mixture:
    experts = cfg.get("num_local_experts") or cfg.get("num_experts")
    return Mixture(experts=int(experts), top_k=int(cfg.get("num_experts_per_tok", 2)),
                   expert_features=int(cfg.get("moe_intermediate_size") or cfg["intermediate_size"]),
                   norm_topk_prob=True if always_norm else bool(cfg.get("norm_topk_prob", True)))


@dataclass(frozen=True)
class Family:
    name: str
    model_types: Tuple[str, ...]
    architecture: str                                     # what ``config.json`` lists under ``architectures`` on export
    read_config: Callable[[Mapping[str, Any]], Dict[str, Any]]
    norm_offset: float = 0.0                              # the release stores ``weight - norm_offset`` (Gemma: 1)
    fused_qkv: Optional[str] = None                       # a single tensor on disk holding q | k | v
    fused_gate_up: Optional[str] = None                   # a single tensor holding gate | up
    qkv_bias: bool = False
    post_attention_norm: str = "post_attention_layernorm"  # the norm in front of the MLP
    mixer_out_norm: Optional[str] = None                  # Gemma-2: norm on the attention output
    mlp_out_norm: Optional[str] = None                    # Gemma-2: norm on the MLP output
    pre_norm: bool = True                                 # False (OLMo-2): no input / pre-MLP norms on disk
    rotary_pairs: bool = False                            # the release rotates pairs (2i, 2i + 1) of a head, not its halves
    experts: Optional[str] = None                         # 'mixtral' | 'qwen' naming of sparse layers
    extra_config: Mapping[str, Any] = field(default_factory=dict)   # written into ``config.json`` on export


def _llama(cfg):
    return _common(cfg, window=cfg.get("sliding_window"))


def _qwen2(cfg):
    use_window = cfg.get("use_sliding_window", False)
    return _common(cfg, qkv_bias=True, window=cfg.get("sliding_window") if use_window else None)


def _dream(cfg):
    """Dream: Qwen2's block read bidirectionally (a masked-diffusion language model)."""
    return dict(_qwen2(cfg), causal=False)


def _qwen3(cfg):
    return _common(cfg, qk_norm=True)


def _qwen3_moe(cfg):
    return _common(cfg, qk_norm=True, mixture=_mixture(cfg, always_norm=False))


def _qwen2_moe(cfg):
    n = cfg["num_hidden_layers"]
    sparse_step, dense_only = int(cfg.get("decoder_sparse_step", 1) or 1), set(cfg.get("mlp_only_layers") or ())
    mix = Mixture(experts=int(cfg["num_experts"]), top_k=int(cfg["num_experts_per_tok"]), expert_features=int(cfg["moe_intermediate_size"]),
                  norm_topk_prob=bool(cfg.get("norm_topk_prob", False)), shared_features=int(cfg.get("shared_expert_intermediate_size") or 0),
                  shared_gate=True, layers=tuple(i for i in range(n) if i not in dense_only and (i + 1) % sparse_step == 0))
    use_window = cfg.get("use_sliding_window", False)
    return _common(cfg, qkv_bias=True, mixture=mix, window=cfg.get("sliding_window") if use_window else None)


def _mixtral(cfg):
    return _common(cfg, window=cfg.get("sliding_window"), mixture=_mixture(cfg, always_norm=True))


def _gemma(cfg):
    act = cfg.get("hidden_activation") or cfg.get("hidden_act") or "gelu_pytorch_tanh"
    return _common(cfg, embed_scale=True, tie_embeddings=True, mlp_activation="gelu_tanh" if "tanh" in act else "gelu")


def _gemma2(cfg):
    base = _gemma(cfg)
    base.update(sandwich_norm=True, attn_softcap=float(cfg.get("attn_logit_softcapping") or 0.0),
                logit_softcap=float(cfg.get("final_logit_softcapping") or 0.0), window=cfg.get("sliding_window"),
                layer_types=("local", "attention"),                 # even layers slide, odd layers see everything
                query_scale=float(cfg.get("query_pre_attn_scalar", base["head_dim"])) ** -0.5)
    return base


def _phi3(cfg):
    return _common(cfg, window=cfg.get("sliding_window"))


def _olmo2(cfg):
    return _common(cfg, pre_norm=False, sandwich_norm=True, qk_norm_full=True)


_KINDS = {"sliding_attention": "local", "full_attention": "attention", "linear_attention": "gdn"}


def _layer_kinds(cfg) -> Optional[Tuple[str, ...]]:
    kinds = cfg.get("layer_types")
    return None if not kinds else tuple(_KINDS[k] for k in kinds)


def _by_kind_rope(cfg) -> Tuple[float, Optional[dict], Optional[float]]:
    """``rope_parameters`` keyed by layer kind (Gemma-3): the full layers' base and scaling, and the sliding layers' base."""
    rope = cfg.get("rope_parameters") or {}
    if "full_attention" in rope:
        full, local = rope["full_attention"], rope.get("sliding_attention") or {}
        scaling = {k: v for k, v in full.items() if k != "rope_theta"} if full.get("rope_type", "default") != "default" else None
        return float(full.get("rope_theta", 10000.0)), scaling, float(local.get("rope_theta", 10000.0))
    theta, scaling = _rope(cfg)
    return theta, scaling, float(cfg.get("rope_local_base_freq", 10000.0))


def _gemma3(cfg):
    base = _gemma(cfg)
    theta, scaling, local = _by_kind_rope(cfg)
    base.update(sandwich_norm=True, qk_norm=True, logit_softcap=float(cfg.get("final_logit_softcapping") or 0.0),
                attn_softcap=float(cfg.get("attn_logit_softcapping") or 0.0), window=cfg.get("sliding_window"),
                layer_types=_layer_kinds(cfg), rope_theta=theta, rope_scaling=scaling, local_rope_theta=local,
                query_scale=float(cfg.get("query_pre_attn_scalar", base["head_dim"])) ** -0.5)
    return base


def _olmo3(cfg):
    # the sliding layers rotate by the plain table; only the full layers take the long-context scaling (the model's paper and the
    # modelling code its release shipped with; later transformers versions build one table for every layer)
    base = _olmo2(cfg)
    base.update(window=cfg.get("sliding_window"), layer_types=_layer_kinds(cfg), local_rope_theta=base["rope_theta"])
    return base


def _smollm3(cfg):
    kinds = _layer_kinds(cfg) or ("attention",) * cfg["num_hidden_layers"]
    rotary = cfg.get("no_rope_layers") or [1] * len(kinds)          # 1: rotary, 0: no positions
    if any(k == "local" and not r for k, r in zip(kinds, rotary)):
        raise NotImplementedError("a sliding layer without rotary positions is not built")
    window = cfg.get("sliding_window") if cfg.get("use_sliding_window") else None
    return _common(cfg, window=window, layer_types=tuple(k if r else "nope" for k, r in zip(kinds, rotary)))


def _deepseek_v3(cfg):
    """Latent attention on every layer; the first ``first_k_dense_replace`` layers dense, the rest routed by sigmoid scores with a selection
    bias inside expert groups, beside always-on shared experts."""
    n = cfg["num_hidden_layers"]
    first, every = int(cfg.get("first_k_dense_replace", 0)), int(cfg.get("moe_layer_freq", 1) or 1)
    width = int(cfg["moe_intermediate_size"])
    mix = Mixture(experts=int(cfg["n_routed_experts"]), top_k=int(cfg["num_experts_per_tok"]),
                  layers=tuple(i for i in range(n) if i >= first and i % every == 0), score_function="sigmoid",
                  norm_topk_prob=bool(cfg.get("norm_topk_prob", True)), scaling=float(cfg.get("routed_scaling_factor", 1.0)), bias=True,
                  groups=int(cfg.get("n_group") or 1), topk_groups=int(cfg.get("topk_group") or 1), expert_features=width,
                  shared_features=int(cfg.get("n_shared_experts") or 0) * width)
    theta, scaling = _rope(cfg)
    gain = 1.0
    if scaling and scaling.get("mscale_all_dim"):                # YaRN: the softmax scale grows by the magnitude correction squared
        f = float(scaling["factor"])
        gain = (1.0 if f <= 1 else 0.1 * float(scaling["mscale_all_dim"]) * math.log(f) + 1.0) ** 2
    options = dict(kv_latent=int(cfg["kv_lora_rank"]), q_latent=cfg.get("q_lora_rank"), nope_dim=int(cfg["qk_nope_head_dim"]),
                   rope_dim=int(cfg["qk_rope_head_dim"]), v_dim=int(cfg["v_head_dim"]), softmax_gain=gain)
    return _common(cfg, head_dim=int(cfg["qk_rope_head_dim"]), layer_types=("mla",), mixture=mix, mixer_options=options)


def _glm4(cfg):
    rope = cfg.get("rope_parameters") or {}
    return _common(cfg, qkv_bias=bool(cfg.get("attention_bias", True)), sandwich_norm=True,
                   rotary_fraction=float(rope.get("partial_rotary_factor", cfg.get("partial_rotary_factor", 0.5))))


def _gpt_oss(cfg):
    mix = Mixture(experts=int(cfg["num_local_experts"]), top_k=int(cfg.get("num_experts_per_tok", 4)), expert_features=int(cfg["intermediate_size"]),
                  style="clamped_glu")
    return _common(cfg, attn_bias=True, attention_sinks=True, window=cfg.get("sliding_window"), layer_types=_layer_kinds(cfg), mixture=mix)


def _qwen3_next(cfg):
    """Gated delta-rule layers with a softmax attention layer every ``full_attention_interval``-th; gated attention outputs; a quarter of
    each head rotating; zero-centred norm weights; routed experts beside a gated shared expert."""
    n = cfg["num_hidden_layers"]
    every = int(cfg.get("full_attention_interval", 4))
    kinds = _layer_kinds(cfg) or tuple("attention" if (i + 1) % every == 0 else "gdn" for i in range(n))
    rope = cfg.get("rope_parameters") or {}
    sparse_step, dense_only = int(cfg.get("decoder_sparse_step", 1) or 1), set(cfg.get("mlp_only_layers") or ())
    mix = Mixture(experts=int(cfg["num_experts"]), top_k=int(cfg["num_experts_per_tok"]), expert_features=int(cfg["moe_intermediate_size"]),
                  norm_topk_prob=bool(cfg.get("norm_topk_prob", True)), shared_features=int(cfg.get("shared_expert_intermediate_size") or 0),
                  shared_gate=True, layers=tuple(i for i in range(n) if i not in dense_only and (i + 1) % sparse_step == 0))
    options = dict(num_k_heads=int(cfg["linear_num_key_heads"]), num_v_heads=int(cfg["linear_num_value_heads"]), head_k_dim=int(cfg["linear_key_head_dim"]),
                   head_v_dim=int(cfg["linear_value_head_dim"]), conv_size=int(cfg.get("linear_conv_kernel_dim", 4)), norm_eps=float(cfg.get("rms_norm_eps", 1e-6)), qk_eps=1e-6)
    return _common(cfg, qk_norm=True, attn_out_gate=True, layer_types=kinds, mixture=mix, mixer_options=options,
                   rotary_fraction=float(rope.get("partial_rotary_factor", cfg.get("partial_rotary_factor", 0.25))))


def _granite(cfg):
    # four scalars: embeddings times one, the softmax scale itself (not 1 / sqrt(d)), every branch times one, logits over one
    return _common(cfg, embed_multiplier=float(cfg.get("embedding_multiplier", 1.0)), query_scale=float(cfg.get("attention_multiplier", 1.0)),
                   residual_multiplier=float(cfg.get("residual_multiplier", 1.0)), logit_divisor=float(cfg.get("logits_scaling", 1.0)))


FAMILIES: Dict[str, Family] = {f.name: f for f in (
    Family("llama", ("llama", "yi"), "LlamaForCausalLM", _llama),
    Family("granite", ("granite",), "GraniteForCausalLM", _granite),
    Family("olmo2", ("olmo2",), "Olmo2ForCausalLM", _olmo2, pre_norm=False, mixer_out_norm="post_attention_layernorm",
           mlp_out_norm="post_feedforward_layernorm"),
    Family("olmo3", ("olmo3",), "Olmo3ForCausalLM", _olmo3, pre_norm=False, mixer_out_norm="post_attention_layernorm",
           mlp_out_norm="post_feedforward_layernorm"),
    Family("smollm3", ("smollm3",), "SmolLM3ForCausalLM", _smollm3),
    Family("mistral", ("mistral",), "MistralForCausalLM", _llama),
    Family("qwen2", ("qwen2",), "Qwen2ForCausalLM", _qwen2, qkv_bias=True),
    Family("dream", ("dream",), "DreamModel", _dream, qkv_bias=True),
    Family("qwen3", ("qwen3",), "Qwen3ForCausalLM", _qwen3),
    Family("qwen3_moe", ("qwen3_moe",), "Qwen3MoeForCausalLM", _qwen3_moe, experts="qwen"),
    Family("qwen2_moe", ("qwen2_moe",), "Qwen2MoeForCausalLM", _qwen2_moe, qkv_bias=True, experts="qwen"),
    Family("mixtral", ("mixtral",), "MixtralForCausalLM", _mixtral, experts="mixtral"),
    Family("gemma", ("gemma",), "GemmaForCausalLM", _gemma, norm_offset=1.0, extra_config={"hidden_activation": "gelu_pytorch_tanh"}),
    Family("gemma2", ("gemma2",), "Gemma2ForCausalLM", _gemma2, norm_offset=1.0, mixer_out_norm="post_attention_layernorm",
           post_attention_norm="pre_feedforward_layernorm", mlp_out_norm="post_feedforward_layernorm",
           extra_config={"hidden_activation": "gelu_pytorch_tanh"}),
    Family("gemma3", ("gemma3_text",), "Gemma3ForCausalLM", _gemma3, norm_offset=1.0, mixer_out_norm="post_attention_layernorm",
           post_attention_norm="pre_feedforward_layernorm", mlp_out_norm="post_feedforward_layernorm",
           extra_config={"hidden_activation": "gelu_pytorch_tanh"}),
    Family("deepseek_v3", ("deepseek_v3",), "DeepseekV3ForCausalLM", _deepseek_v3, experts="deepseek"),
    Family("glm4", ("glm4",), "Glm4ForCausalLM", _glm4, qkv_bias=True, rotary_pairs=True, fused_gate_up="mlp.gate_up_proj",
           mixer_out_norm="post_self_attn_layernorm", mlp_out_norm="post_mlp_layernorm"),
    Family("gpt_oss", ("gpt_oss",), "GptOssForCausalLM", _gpt_oss, qkv_bias=True, experts="gpt_oss"),
    Family("qwen3_next", ("qwen3_next",), "Qwen3NextForCausalLM", _qwen3_next, norm_offset=1.0, experts="qwen3_next"),
    Family("phi3", ("phi3",), "Phi3ForCausalLM", _phi3, fused_qkv="self_attn.qkv_proj", fused_gate_up="mlp.gate_up_proj"),
)}


def family_of(cfg: Mapping[str, Any]) -> Family:
    """The family a ``config.json`` belongs to: by ``model_type`` first, else by the first entry of ``architectures``."""
    mt = str(cfg.get("model_type") or "").lower()
    for fam in FAMILIES.values():
        if mt in fam.model_types:
            return fam
    arch = (cfg.get("architectures") or [""])[0].lower()
    best = None
    for fam in FAMILIES.values():                              # longest matching name wins: qwen3_moe before qwen3
        key = fam.name.replace("_", "")
        if key in arch and (best is None or len(key) > len(best.name.replace("_", ""))):
            best = fam
    if best is None:
        raise KeyError(f"no decoder family for model_type {mt!r} / architectures {cfg.get('architectures')}; known: {sorted(FAMILIES)}")
    return best


def read_config(cfg: Mapping[str, Any]) -> TransformerConfig:
    return TransformerConfig(**family_of(cfg).read_config(cfg))


def write_config(c: TransformerConfig, family: str = "llama", dtype: str = "bfloat16") -> Dict[str, Any]:
    fam = FAMILIES[family]
    rope = {"rope_theta": c.rope_theta, "rope_type": "default"} if not c.rope_scaling else {"rope_theta": c.rope_theta, **c.rope_scaling}
    out = {"model_type": fam.model_types[0], "architectures": [fam.architecture], "vocab_size": c.vocab_size, "hidden_size": c.emb_features,
           "num_hidden_layers": c.num_layers, "num_attention_heads": c.num_heads, "num_key_value_heads": c.num_kv_heads or c.num_heads,
           "head_dim": c.head_dim or c.emb_features // c.num_heads, "intermediate_size": c.mlp_features,
           "max_position_embeddings": c.max_seq_len, "rope_theta": c.rope_theta, "rope_scaling": c.rope_scaling, "rope_parameters": rope,
           "rms_norm_eps": c.norm_eps, "tie_word_embeddings": c.tie_embeddings, "hidden_act": "silu", "torch_dtype": dtype, "dtype": dtype,
           "sliding_window": c.window, **fam.extra_config}
    if c.mixture is not None:
        m = c.mixture
        out.update({"num_experts": m.experts, "num_local_experts": m.experts, "num_experts_per_tok": m.top_k, "norm_topk_prob": m.norm_topk_prob,
                    "moe_intermediate_size": m.expert_features or c.mlp_features, "decoder_sparse_step": 1, "mlp_only_layers": []})
    if fam.name == "gemma2":
        out.update({"attn_logit_softcapping": c.attn_softcap or None, "final_logit_softcapping": c.logit_softcap or None,
                    "query_pre_attn_scalar": (c.query_scale ** -2) if c.query_scale else out["head_dim"]})
    kinds = c.kinds()
    if fam.name in ("gemma3", "olmo3", "smollm3", "gpt_oss"):
        out["layer_types"] = ["sliding_attention" if k == "local" else "full_attention" for k in kinds]
    if fam.name == "gemma3":
        full = {"rope_type": "default", **(c.rope_scaling or {}), "rope_theta": c.rope_theta}
        out.update({"query_pre_attn_scalar": (c.query_scale ** -2) if c.query_scale else out["head_dim"],
                    "final_logit_softcapping": c.logit_softcap or None, "attn_logit_softcapping": c.attn_softcap or None,
                    "rope_parameters": {"full_attention": full, "sliding_attention": {"rope_type": "default", "rope_theta": c.local_rope_theta or 10000.0}}})
        out.pop("rope_theta"), out.pop("rope_scaling")
    if fam.name == "smollm3":
        out.update({"no_rope_layers": [0 if k == "nope" else 1 for k in kinds], "use_sliding_window": c.window is not None})
    if fam.name == "deepseek_v3":
        m, o = c.mixture, c.mixer_options
        sparse = sorted(m.layers) if m.layers is not None else list(range(c.num_layers))
        if sparse != list(range(sparse[0] if sparse else c.num_layers, c.num_layers)):
            raise ValueError("a DeepSeek-V3 release says which layers are sparse by the count of dense layers in front of them")
        out.update({"n_routed_experts": m.experts, "n_shared_experts": m.shared_features // (m.expert_features or 1), "n_group": m.groups,
                    "topk_group": m.topk_groups, "routed_scaling_factor": m.scaling, "first_k_dense_replace": sparse[0] if sparse else c.num_layers,
                    "moe_layer_freq": 1, "kv_lora_rank": o["kv_latent"], "q_lora_rank": o.get("q_latent"), "qk_nope_head_dim": o["nope_dim"],
                    "qk_rope_head_dim": o["rope_dim"], "v_head_dim": o["v_dim"], "head_dim": o["rope_dim"],
                    "num_key_value_heads": c.num_heads, "rope_interleave": True})
    if fam.name == "qwen2_moe":
        out.update({"shared_expert_intermediate_size": c.mixture.shared_features, "use_sliding_window": c.window is not None})
    if fam.name == "qwen3_next":
        o, m = c.mixer_options, c.mixture
        out.update({"layer_types": ["linear_attention" if k == "gdn" else "full_attention" for k in kinds], "linear_num_key_heads": o["num_k_heads"],
                    "linear_num_value_heads": o["num_v_heads"], "linear_key_head_dim": o["head_k_dim"], "linear_value_head_dim": o["head_v_dim"],
                    "linear_conv_kernel_dim": o.get("conv_size", 4), "shared_expert_intermediate_size": m.shared_features,
                    "partial_rotary_factor": c.rotary_fraction, "rope_parameters": {**out["rope_parameters"], "partial_rotary_factor": c.rotary_fraction},
                    "full_attention_interval": next((i + 1 for i, k in enumerate(kinds) if k != "gdn"), len(kinds) + 1)})
    if fam.name == "glm4":
        out.update({"attention_bias": c.qkv_bias, "partial_rotary_factor": c.rotary_fraction})
        out["rope_parameters"] = {**out["rope_parameters"], "partial_rotary_factor": c.rotary_fraction}
    if fam.name == "qwen2":
        out["use_sliding_window"] = c.window is not None
    if fam.name == "granite":
        hd = out["head_dim"]
        out.update({"embedding_multiplier": c.embed_multiplier if c.embed_multiplier is not None else 1.0,
                    "attention_multiplier": c.query_scale if c.query_scale is not None else hd ** -0.5,
                    "residual_multiplier": c.residual_multiplier, "logits_scaling": c.logit_divisor})
    return out


# ------------------------------------------------------------------------------------------------ tensors
class _Indexed:
    """A reader behind ``[]`` (for the layer loaders that index a mapping)."""

    def __init__(self, get):
        self.get = get

    def __getitem__(self, key):
        return self.get(key)

    def __contains__(self, key):
        return self.get.has(key)


class _Reader:
    """A release's tensors with a record of which were read."""

    def __init__(self, tensors: Mapping[str, torch.Tensor]):
        self.tensors, self.read = tensors, set()

    def __call__(self, key: str) -> torch.Tensor:
        self.read.add(key)
        return self.tensors[key]

    def has(self, key: str) -> bool:
        return key in self.tensors

    def unread(self) -> List[str]:
        return sorted(k for k in self.tensors if k not in self.read and not k.endswith("rotary_emb.inv_freq"))


def _put(p: torch.Tensor, t: torch.Tensor, offset: float = 0.0) -> None:
    if tuple(p.shape) != tuple(t.shape):
        raise ValueError(f"shape {tuple(t.shape)} on disk does not fit the parameter's {tuple(p.shape)}")
    with torch.no_grad():
        p.copy_((t.float() + offset).to(p.dtype) if offset else t.to(p.dtype))


def load_state(model: CausalTransformer, tensors: Mapping[str, torch.Tensor], family: Family, strict: bool = True) -> List[str]:
    """Copy a release's tensors into ``model``; returns the keys of ``tensors`` nothing read (raises on them with ``strict``)."""
    get = _Reader(tensors)
    off = family.norm_offset
    c = model.config
    H, Hkv = c.num_heads, c.num_kv_heads or c.num_heads
    D = c.head_dim or c.emb_features // c.num_heads
    _put(model.embed.weight, get("model.embed_tokens.weight"))
    for i, layer in enumerate(model.layers):
        pre = f"model.layers.{i}."
        if family.pre_norm:
            _put(layer.input_norm.weight, get(pre + "input_layernorm.weight"), off)
            _put(layer.post_norm.weight, get(pre + family.post_attention_norm + ".weight"), off)
        if family.mixer_out_norm:
            _put(layer.mixer_out_norm.weight, get(pre + family.mixer_out_norm + ".weight"), off)
            _put(layer.mlp_out_norm.weight, get(pre + family.mlp_out_norm + ".weight"), off)
        a = layer.mixer
        if hasattr(a, "kv_latent"):
            _load_latent_attention(a, get, pre + "self_attn.")
        elif hasattr(a, "in_proj_qkvz"):
            from .hf import load_gated_delta_net
            load_gated_delta_net(a, _Indexed(get), pre + "linear_attn.")
        elif getattr(a, "gate_proj", None) is not None:
            # the query projection holds, per head, the query then its output gate
            order = head_order(a.head_dim, int(a.head_dim * model.config.rotary_fraction), family.rotary_pairs)
            H, Hkv, D = a.num_heads, a.num_kv_heads, a.head_dim
            qg = get(pre + "self_attn.q_proj.weight").reshape(H, 2 * D, -1)
            packed = torch.cat([qg[:, :D].reshape(H * D, -1), get(pre + "self_attn.k_proj.weight"), get(pre + "self_attn.v_proj.weight")], 0)
            _put(a.qkv_proj.weight, _reorder_qk(packed, H, Hkv, D, order))
            _put(a.gate_proj.weight, qg[:, D:].reshape(H * D, -1))
            _put(a.o_proj.weight, get(pre + "self_attn.o_proj.weight"))
            _put(a.q_norm.weight, get(pre + "self_attn.q_norm.weight")[order] if order is not None else get(pre + "self_attn.q_norm.weight"), off)
            _put(a.k_norm.weight, get(pre + "self_attn.k_norm.weight")[order] if order is not None else get(pre + "self_attn.k_norm.weight"), off)
        else:
            order = head_order(a.head_dim, int(a.head_dim * model.config.rotary_fraction), family.rotary_pairs)
            shape = (a.num_heads, a.num_kv_heads, a.head_dim, order)
            if family.fused_qkv:
                _put(a.qkv_proj.weight, _reorder_qk(get(pre + family.fused_qkv + ".weight"), *shape))
            else:
                _put(a.qkv_proj.weight, _reorder_qk(torch.cat([get(pre + f"self_attn.{n}_proj.weight") for n in "qkv"], 0), *shape))
            if a.qkv_proj.bias is not None:
                _put(a.qkv_proj.bias, _reorder_qk(torch.cat([get(pre + f"self_attn.{n}_proj.bias") for n in "qkv"], 0), *shape))
            _put(a.o_proj.weight, get(pre + "self_attn.o_proj.weight"))
            if a.o_proj.bias is not None:
                _put(a.o_proj.bias, get(pre + "self_attn.o_proj.bias"))
            if a.sinks is not None:
                _put(a.sinks, get(pre + "self_attn.sinks"))
            if a.q_norm is not None:
                _put(a.q_norm.weight, get(pre + "self_attn.q_norm.weight"), off)
                _put(a.k_norm.weight, get(pre + "self_attn.k_norm.weight"), off)
        if getattr(layer, "sparse", False) and family.experts == "gpt_oss":
            _load_clamped_glu(layer.mlp, get, pre + "mlp.")
        elif getattr(layer, "sparse", False):
            _load_experts(layer.mlp, get, pre)
        elif family.fused_gate_up:
            _put(layer.mlp.gate_up_proj.weight, get(pre + family.fused_gate_up + ".weight"))
            _put(layer.mlp.down_proj.weight, get(pre + "mlp.down_proj.weight"))
        else:
            _put(layer.mlp.gate_up_proj.weight, torch.cat([get(pre + "mlp.gate_proj.weight"), get(pre + "mlp.up_proj.weight")], 0))
            _put(layer.mlp.down_proj.weight, get(pre + "mlp.down_proj.weight"))
    _put(model.final_norm.weight, get("model.norm.weight"), off)
    if model.head is not None:
        _put(model.head.weight, get("lm_head.weight") if get.has("lm_head.weight") else get("model.embed_tokens.weight"))
    elif get.has("lm_head.weight"):
        get.read.add("lm_head.weight")                          # a tied release may still store the copy
    left = get.unread()
    if strict and left:
        raise KeyError(f"{len(left)} tensor(s) of the release were not read by the {family.name} mapping: {left[:6]}")
    return left


def head_order(D: int, R: int, pairs: bool) -> Optional[torch.Tensor]:
    """Where each dimension of a head as this library lays it out, ``[rotated a | kept a | rotated b | kept b]``, sits in the release's
    head, which rotates its first ``R`` dimensions as pairs ``(2i, 2i + 1)`` or as halves ``(i, i + R / 2)``.  None: the same order."""
    if R >= D and not pairs:
        return None
    a, b = (torch.arange(0, R, 2), torch.arange(1, R, 2)) if pairs else (torch.arange(0, R // 2), torch.arange(R // 2, R))
    keep = (D - R) // 2
    return torch.cat([a, torch.arange(R, R + keep), b, torch.arange(R + keep, D)])


def _reorder_qk(t: torch.Tensor, H: int, Hkv: int, D: int, order: Optional[torch.Tensor], back: bool = False) -> torch.Tensor:
    """Rows of a packed q | k | v weight or bias with every q and k head's dimensions reordered (``back``: undone)."""
    if order is None:
        return t
    idx = torch.argsort(order) if back else order
    heads = t.reshape(H + 2 * Hkv, D, -1).clone()
    heads[: H + Hkv] = heads[: H + Hkv][:, idx]
    return heads.reshape(t.shape)


def _pairs_to_halves(rope: int) -> torch.Tensor:
    """DeepSeek stores a rotary vector as pairs ``(2i, 2i + 1)``; this library rotates halves ``(i, i + rope / 2)``."""
    return torch.cat([torch.arange(0, rope, 2), torch.arange(1, rope, 2)])


def _load_latent_attention(a, get: _Reader, pre: str) -> None:
    H, nope, rope = a.h, a.nope, a.rope
    perm = _pairs_to_halves(rope)
    if a.q_down is not None:
        _put(a.q_down.weight, get(pre + "q_a_proj.weight"))
        _put(a.q_norm.weight, get(pre + "q_a_layernorm.weight"))
        q = get(pre + "q_b_proj.weight")
    else:
        q = get(pre + "q_proj.weight")
    q = q.reshape(H, nope + rope, -1).clone()
    q[:, nope:] = q[:, nope:][:, perm]
    _put(a.q_up.weight, q.reshape(H * (nope + rope), -1))
    kv = get(pre + "kv_a_proj_with_mqa.weight").clone()
    kv[-rope:] = kv[-rope:][perm]
    _put(a.kv_down.weight, kv)
    _put(a.kv_norm.weight, get(pre + "kv_a_layernorm.weight"))
    _put(a.kv_up.weight, get(pre + "kv_b_proj.weight"))
    _put(a.o_proj.weight, get(pre + "o_proj.weight"))


def _export_latent_attention(a, out: Dict[str, torch.Tensor], pre: str) -> None:
    H, nope, rope = a.h, a.nope, a.rope
    back = torch.argsort(_pairs_to_halves(rope))
    q = a.q_up.weight.detach().reshape(H, nope + rope, -1).clone()
    q[:, nope:] = q[:, nope:][:, back]
    q = q.reshape(H * (nope + rope), -1)
    if a.q_down is not None:
        out[pre + "q_a_proj.weight"], out[pre + "q_a_layernorm.weight"], out[pre + "q_b_proj.weight"] = a.q_down.weight.detach(), a.q_norm.weight.detach(), q
    else:
        out[pre + "q_proj.weight"] = q
    kv = a.kv_down.weight.detach().clone()
    kv[-rope:] = kv[-rope:][back]
    out[pre + "kv_a_proj_with_mqa.weight"], out[pre + "kv_a_layernorm.weight"] = kv, a.kv_norm.weight.detach()
    out[pre + "kv_b_proj.weight"], out[pre + "o_proj.weight"] = a.kv_up.weight.detach(), a.o_proj.weight.detach()


def _load_clamped_glu(mlp, get: _Reader, pre: str) -> None:
    """GPT-OSS stores ``gate_up_proj [E, d, 2F]`` input-major with gate and linear columns interleaved, ``down_proj [E, F, d]``."""
    _put(mlp.router.weight, get(pre + "router.weight"))
    _put(mlp.router.bias, get(pre + "router.bias"))
    gu, gb = get(pre + "experts.gate_up_proj"), get(pre + "experts.gate_up_proj_bias")
    _put(mlp.experts.gate_up, torch.cat([gu[..., 0::2], gu[..., 1::2]], -1).transpose(1, 2))
    _put(mlp.experts.gate_up_bias, torch.cat([gb[..., 0::2], gb[..., 1::2]], -1))
    _put(mlp.experts.down, get(pre + "experts.down_proj").transpose(1, 2))
    _put(mlp.experts.down_bias, get(pre + "experts.down_proj_bias"))


def _export_clamped_glu(mlp, out: Dict[str, torch.Tensor], pre: str) -> None:
    out[pre + "router.weight"], out[pre + "router.bias"] = mlp.router.weight.detach(), mlp.router.bias.detach()
    gu, gb = mlp.experts.gate_up.detach().transpose(1, 2), mlp.experts.gate_up_bias.detach()       # [E, d, 2F] halves, [E, 2F]
    Fh = gb.shape[-1] // 2
    out[pre + "experts.gate_up_proj"] = torch.stack([gu[..., :Fh], gu[..., Fh:]], -1).flatten(-2)
    out[pre + "experts.gate_up_proj_bias"] = torch.stack([gb[..., :Fh], gb[..., Fh:]], -1).flatten(-2)
    out[pre + "experts.down_proj"] = mlp.experts.down.detach().transpose(1, 2)
    out[pre + "experts.down_proj_bias"] = mlp.experts.down_bias.detach()


def _load_experts(mlp, get: _Reader, pre: str) -> None:
    E = mlp.mix.experts
    if get.has(pre + "mlp.gate.e_score_correction_bias"):
        _put(mlp.router.expert_bias, get(pre + "mlp.gate.e_score_correction_bias"))
    if mlp.shared is not None and get.has(pre + "mlp.shared_expert.gate_proj.weight"):             # Qwen3-Next / Qwen2-MoE: one gated shared expert
        _put(mlp.shared.gate_up_proj.weight, torch.cat([get(pre + "mlp.shared_expert.gate_proj.weight"), get(pre + "mlp.shared_expert.up_proj.weight")], 0))
        _put(mlp.shared.down_proj.weight, get(pre + "mlp.shared_expert.down_proj.weight"))
        if mlp.shared_gate is not None:
            _put(mlp.shared_gate.weight, get(pre + "mlp.shared_expert_gate.weight"))
    if mlp.shared is not None and get.has(pre + "mlp.shared_experts.gate_proj.weight"):
        _put(mlp.shared.gate_up_proj.weight, torch.cat([get(pre + "mlp.shared_experts.gate_proj.weight"), get(pre + "mlp.shared_experts.up_proj.weight")], 0))
        _put(mlp.shared.down_proj.weight, get(pre + "mlp.shared_experts.down_proj.weight"))
    for gate in ("mlp.gate.weight", "block_sparse_moe.gate.weight"):
        if get.has(pre + gate):
            _put(mlp.router.weight, get(pre + gate))
            break
    else:
        raise KeyError(f"no router weight under {pre}")
    if get.has(pre + "mlp.experts.gate_up_proj"):
        _put(mlp.experts.gate_up, get(pre + "mlp.experts.gate_up_proj"))
        _put(mlp.experts.down, get(pre + "mlp.experts.down_proj"))
        return
    if get.has(pre + "block_sparse_moe.experts.0.w1.weight"):
        names = ("block_sparse_moe.experts.{}.w1.weight", "block_sparse_moe.experts.{}.w3.weight", "block_sparse_moe.experts.{}.w2.weight")
    else:
        names = ("mlp.experts.{}.gate_proj.weight", "mlp.experts.{}.up_proj.weight", "mlp.experts.{}.down_proj.weight")
    _put(mlp.experts.gate_up, torch.stack([torch.cat([get(pre + names[0].format(j)), get(pre + names[1].format(j))], 0) for j in range(E)]))
    _put(mlp.experts.down, torch.stack([get(pre + names[2].format(j)) for j in range(E)]))


def export_state(model: CausalTransformer, family: Family) -> Dict[str, torch.Tensor]:
    """The model's tensors under the names and layouts ``family``'s releases use."""
    c = model.config
    H, Hkv = c.num_heads, c.num_kv_heads or c.num_heads
    D = c.head_dim or c.emb_features // c.num_heads
    off = family.norm_offset

    def norm(p):
        return (p.detach().float() - off).to(p.dtype) if off else p.detach()
    out = {"model.embed_tokens.weight": model.embed.weight.detach(), "model.norm.weight": norm(model.final_norm.weight)}
    for i, layer in enumerate(model.layers):
        pre = f"model.layers.{i}."
        if family.pre_norm:
            out[pre + "input_layernorm.weight"] = norm(layer.input_norm.weight)
            out[pre + family.post_attention_norm + ".weight"] = norm(layer.post_norm.weight)
        if family.mixer_out_norm:
            out[pre + family.mixer_out_norm + ".weight"] = norm(layer.mixer_out_norm.weight)
            out[pre + family.mlp_out_norm + ".weight"] = norm(layer.mlp_out_norm.weight)
        a = layer.mixer
        if hasattr(a, "kv_latent"):
            _export_latent_attention(a, out, pre + "self_attn.")
        elif hasattr(a, "in_proj_qkvz"):
            from .hf import export_gated_delta_net
            export_gated_delta_net(a, out, pre + "linear_attn.")
        elif getattr(a, "gate_proj", None) is not None:
            order = head_order(D, int(D * c.rotary_fraction), family.rotary_pairs)
            w = _reorder_qk(a.qkv_proj.weight.detach(), H, Hkv, D, order, back=True)
            qg = torch.cat([w[: H * D].reshape(H, D, -1), a.gate_proj.weight.detach().reshape(H, D, -1)], 1)
            out[pre + "self_attn.q_proj.weight"] = qg.reshape(2 * H * D, -1)
            out[pre + "self_attn.k_proj.weight"], out[pre + "self_attn.v_proj.weight"] = w[H * D:(H + Hkv) * D], w[(H + Hkv) * D:]
            out[pre + "self_attn.o_proj.weight"] = a.o_proj.weight.detach()
            back = torch.argsort(order) if order is not None else slice(None)
            out[pre + "self_attn.q_norm.weight"], out[pre + "self_attn.k_norm.weight"] = norm(a.q_norm.weight)[back], norm(a.k_norm.weight)[back]
        else:
            order = head_order(D, int(D * c.rotary_fraction), family.rotary_pairs)
            w = _reorder_qk(a.qkv_proj.weight.detach(), H, Hkv, D, order, back=True)
            if family.fused_qkv:
                out[pre + family.fused_qkv + ".weight"] = w
            else:
                for n, part in zip("qkv", (w[: H * D], w[H * D:(H + Hkv) * D], w[(H + Hkv) * D:])):
                    out[pre + f"self_attn.{n}_proj.weight"] = part
            if a.qkv_proj.bias is not None:
                b = _reorder_qk(a.qkv_proj.bias.detach(), H, Hkv, D, order, back=True)
                for n, part in zip("qkv", (b[: H * D], b[H * D:(H + Hkv) * D], b[(H + Hkv) * D:])):
                    out[pre + f"self_attn.{n}_proj.bias"] = part
            out[pre + "self_attn.o_proj.weight"] = a.o_proj.weight.detach()
            if a.o_proj.bias is not None:
                out[pre + "self_attn.o_proj.bias"] = a.o_proj.bias.detach()
            if a.sinks is not None:
                out[pre + "self_attn.sinks"] = a.sinks.detach()
            if a.q_norm is not None:
                out[pre + "self_attn.q_norm.weight"] = norm(a.q_norm.weight)
                out[pre + "self_attn.k_norm.weight"] = norm(a.k_norm.weight)
        if getattr(layer, "sparse", False) and family.experts == "deepseek":
            m = layer.mlp
            out[pre + "mlp.gate.e_score_correction_bias"] = m.router.expert_bias.detach()
            if m.shared is not None:
                sw = m.shared.gate_up_proj.weight.detach()
                out[pre + "mlp.shared_experts.gate_proj.weight"], out[pre + "mlp.shared_experts.up_proj.weight"] = sw[: sw.shape[0] // 2], sw[sw.shape[0] // 2:]
                out[pre + "mlp.shared_experts.down_proj.weight"] = m.shared.down_proj.weight.detach()
        if getattr(layer, "sparse", False) and family.experts == "gpt_oss":
            _export_clamped_glu(layer.mlp, out, pre + "mlp.")
            continue
        if getattr(layer, "sparse", False) and family.experts == "qwen3_next":
            m = layer.mlp
            out[pre + "mlp.gate.weight"] = m.router.weight.detach()
            out[pre + "mlp.experts.gate_up_proj"], out[pre + "mlp.experts.down_proj"] = m.experts.gate_up.detach(), m.experts.down.detach()
            if m.shared is not None:
                sw = m.shared.gate_up_proj.weight.detach()
                out[pre + "mlp.shared_expert.gate_proj.weight"], out[pre + "mlp.shared_expert.up_proj.weight"] = sw[: sw.shape[0] // 2], sw[sw.shape[0] // 2:]
                out[pre + "mlp.shared_expert.down_proj.weight"] = m.shared.down_proj.weight.detach()
                out[pre + "mlp.shared_expert_gate.weight"] = m.shared_gate.weight.detach()
            continue
        if getattr(layer, "sparse", False):
            gu_all, dn_all = layer.mlp.experts.gate_up.detach(), layer.mlp.experts.down.detach()
            Fe = gu_all.shape[1] // 2
            mixtral = family.experts == "mixtral"
            out[pre + ("block_sparse_moe.gate.weight" if mixtral else "mlp.gate.weight")] = layer.mlp.router.weight.detach()
            if layer.mlp.shared is not None and getattr(layer.mlp, "shared_gate", None) is not None:
                sw = layer.mlp.shared.gate_up_proj.weight.detach()
                out[pre + "mlp.shared_expert.gate_proj.weight"], out[pre + "mlp.shared_expert.up_proj.weight"] = sw[: sw.shape[0] // 2], sw[sw.shape[0] // 2:]
                out[pre + "mlp.shared_expert.down_proj.weight"] = layer.mlp.shared.down_proj.weight.detach()
                out[pre + "mlp.shared_expert_gate.weight"] = layer.mlp.shared_gate.weight.detach()
            for j in range(gu_all.shape[0]):
                base = pre + (f"block_sparse_moe.experts.{j}." if mixtral else f"mlp.experts.{j}.")
                g_n, u_n, d_n = ("w1", "w3", "w2") if mixtral else ("gate_proj", "up_proj", "down_proj")
                out[base + g_n + ".weight"], out[base + u_n + ".weight"], out[base + d_n + ".weight"] = gu_all[j, :Fe], gu_all[j, Fe:], dn_all[j]
            continue
        gu = layer.mlp.gate_up_proj.weight.detach()
        if family.fused_gate_up:
            out[pre + family.fused_gate_up + ".weight"] = gu
        else:
            F_ = gu.shape[0] // 2
            out[pre + "mlp.gate_proj.weight"], out[pre + "mlp.up_proj.weight"] = gu[:F_], gu[F_:]
        out[pre + "mlp.down_proj.weight"] = layer.mlp.down_proj.weight.detach()
    if model.head is not None:
        out["lm_head.weight"] = model.head.weight.detach()
    return {k: v.contiguous() for k, v in out.items()}
