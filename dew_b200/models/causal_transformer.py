"""``CausalTransformer``: decoder-only LM backbone - dense (Llama / Qwen / Gemma style), MoE, and hybrid stacks that
interleave attention with gated-delta-net or Mamba-2 mixers.

Fields follow the reference (src/dew/nn/backbones/causal_transformer.py:165-423): ``emb_features, num_layers,
num_heads, num_kv_heads, head_dim, mlp_features, max_seq_len, rope_theta / rope_scaling, layer_types, norm_eps,
qk_norm, tie_embeddings, attention_sinks, softcaps, mixture (MoE), remat``.  Forward structure (reference call
stack, causal_transformer.py:1044-): embed -> per layer [stream RMSNorm -> mixer -> stream RMSNorm -> MLP | MoE]
-> final norm -> head.  The residual add is fused into the next norm (one pass emits both the new stream and its
normalised value).
"""
from __future__ import annotations

import contextlib

from dataclasses import dataclass, field
from typing import Mapping, Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.utils.checkpoint as ckpt

from .. import ops
from ..nn.attention import SelfAttention
from ..nn.layers import Embedding, Linear, RMSNorm
from ..nn.mlp import SwiGLU
from ..utils.registry import register


@dataclass
class Mixture:
    """MoE description (reference: docs/concepts/moe.md:37-57)."""
    experts: int = 8
    top_k: int = 2
    layers: Optional[Sequence[int]] = None          # which layers are sparse (None = all)
    score_function: str = "softmax"                  # softmax | sigmoid
    norm_topk_prob: bool = True
    scaling: float = 1.0
    bias: bool = False                               # aux-loss-free balancing bias (selection only)
    expert_features: Optional[int] = None
    shared_features: int = 0                         # total hidden width of the shared experts
    shared_gate: bool = False
    implementation: str = "auto"
    dispatch: str = "auto"                           # auto | global | exchange
    capacity_factor: Optional[float] = None
    fp8: Any = False                                 # True: block-scaled MXFP8 expert GEMMs (1 x 32 blocks); 'row': row / channel scaled e4m3
    balance_rate: float = 1e-3
    groups: int = 1                                  # DeepSeek-V3's group-limited routing: experts in ``groups`` groups ...
    topk_groups: int = 1                             # ... of which each token may use the ``topk_groups`` best (by their top-2 sum)
    style: str = "swiglu"                            # 'clamped_glu': GPT-OSS's biased router over the top logits and biased clamped-GLU experts


@dataclass(frozen=True)
class Loop:
    """A looped decoder: the layers ``[first, end)`` run ``steps`` times, each pass reading the last one's output, between the layers
    before them (run once) and the coda after them (run once on the exit).  ``exit_gate`` adds a per-token gate on every pass's
    exit state whose hazards give the probability of stopping there (trained by ``LMObjective(exit_entropy=...)``); the passes
    before the last ``backprop_steps`` carry no gradient.  Reference: src/dew/nn/backbones/looping.py (``Loop``)."""
    steps: int = 2
    first: int = 0
    end: Optional[int] = None
    exit_gate: bool = False
    backprop_steps: Optional[int] = None
    messages: int = 0                # n > 0: cross-pass messages - every pass starts from the prelude's output and reads the summaries the pass
    message_rank: int = 16           # before left of every block of n looped layers, merged into each sub-layer's input (nn/cross_pass.py)

    def __post_init__(self):
        if self.steps < 1 or self.first < 0 or (self.end is not None and self.end <= self.first):
            raise ValueError("a loop runs layers [first, end) at least once")
        if self.backprop_steps is not None and not 1 <= self.backprop_steps <= self.steps:
            raise ValueError("backprop_steps counts the last passes that carry a gradient: between 1 and steps")


@dataclass
class TransformerConfig:
    vocab_size: int = 32000
    emb_features: int = 512
    num_layers: int = 8
    num_heads: int = 8
    num_kv_heads: Optional[int] = None
    head_dim: Optional[int] = None
    mlp_features: Optional[int] = None
    max_seq_len: int = 2048
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    norm_eps: float = 1e-6
    qk_norm: bool = True
    tie_embeddings: bool = True
    attention_sinks: bool = False
    attn_softcap: float = 0.0
    logit_softcap: float = 0.0
    window: Optional[int] = None
    layer_types: Optional[Sequence[str]] = None      # per layer: attention | local | nope | gdn | mamba2 | mamba | mamba3 | kda | mla | lightning | differential | forgetting | gla | delta | rwkv7 | memory | none
    mixture: Optional[Mixture] = None
    mixer_options: Dict[str, Any] = field(default_factory=dict)
    remat: bool = False
    init_std: float = 0.02
    embed_scale: bool = False                         # Gemma: multiply embeddings by sqrt(d)
    mtp_depth: int = 0                                # multi-token prediction: extra sequential heads for tokens t+2, t+3, ...
    hyper_connections: int = 0                        # n > 1: n residual streams with learned read / write weights per sub-layer
    altup: int = 0                                    # K > 1: AltUp - K blocks, one of which every sub-layer computes on
    qkv_bias: bool = False                            # Qwen2: bias on the fused q | k | v projection only
    causal: bool = True                               # False: every token sees the whole row (masked-diffusion decoders: LLaDA, Dream)
    attn_out_gate: bool = False                       # Qwen3-Next: a sigmoid gate from the layer's input on the heads' outputs
    attn_bias: bool = False                           # GPT-OSS: bias on q | k | v and on the output projection
    mlp_activation: str = "silu"                      # silu (SwiGLU) | gelu_tanh (Gemma's GeGLU) | gelu
    sandwich_norm: bool = False                       # Gemma-2: every sub-layer's output is normalised before it joins the stream
    query_scale: Optional[float] = None               # softmax scale other than head_dim ** -0.5 (Gemma-2's query_pre_attn_scalar ** -0.5)
    loop: Optional[Loop] = None                       # a block of layers run several times (a looped / recurrent-depth decoder)
    local_rope_theta: Optional[float] = None          # Gemma-3 / OLMo-3: 'local' layers rotate by this base, unscaled; the others by rope_theta with rope_scaling
    rotary_fraction: float = 1.0                      # GLM / Phi / NeoX: only this share of a head's width rotates; heads are laid out [rotated a | kept a | rotated b | kept b]
    layer_mlp: Optional[Sequence[bool]] = None        # per layer (cycled like layer_types): False - the layer is its mixer alone (Mamba's blocks); with the
                                                      # mixer kind 'none', a layer that is its MLP alone (Nemotron-H's and Jamba's separate blocks)
    depth_residual_block: int = 0                     # n > 0: block attention residuals - sub-layers read a learned softmax over the finished blocks of n layers and the partial sum
    engram: Optional[Dict[str, Any]] = None           # {'layers': [i, ...], **Engram fields}: hashed n-gram memories gated into the stream in front of those layers
    pre_norm: bool = True                             # False (OLMo-2): sub-layers read the stream as it is; only their outputs are normalised (sandwich_norm)
    qk_norm_full: bool = False                        # OLMo-2: q and k normalised over all heads at once
    embed_multiplier: Optional[float] = None          # Granite: embeddings times this (embed_scale is the sqrt(d) special case)
    residual_multiplier: float = 1.0                  # Granite: every sub-layer's output times this before it joins the stream
    logit_divisor: float = 1.0                        # Granite: logits divided by this

    def __post_init__(self):
        if isinstance(self.mixture, Mapping):             # a run record (JSON) carries the mixture as a plain mapping
            self.mixture = Mixture(**self.mixture)
        if isinstance(self.loop, Mapping):
            self.loop = Loop(**self.loop)

    def kinds(self) -> List[str]:
        if self.layer_types is None:
            return ["attention"] * self.num_layers
        pattern = list(self.layer_types)
        return [pattern[i % len(pattern)] for i in range(self.num_layers)]


ROTARY_KINDS = ("attention", "local", "nope", "mla", "differential", "forgetting")      # mixers called with the rotary tables and positions


def _mixer(cfg: TransformerConfig, kind: str, dtype, device, index: int = 0) -> nn.Module:
    if kind in ("attention", "local", "nope"):
        a = SelfAttention(cfg.emb_features, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, qk_norm=cfg.qk_norm,
                          causal=cfg.causal, window=cfg.window if kind == "local" or cfg.layer_types is None else None, bias=cfg.attn_bias,
                          softcap=cfg.attn_softcap, sinks=cfg.attention_sinks, norm_eps=cfg.norm_eps,
                          init_std=cfg.init_std, qkv_bias=cfg.qkv_bias, scale=cfg.query_scale, qk_norm_full=cfg.qk_norm_full,
                          out_gate=cfg.attn_out_gate, dtype=dtype, device=device)
        a.rotary = kind != "nope"                        # SmolLM3's every fourth layer attends without positions
        if kind == "local" and cfg.local_rope_theta is not None:
            a.own_rope = (float(cfg.local_rope_theta), None)
        return a
    if kind == "gdn":
        from ..nn.linear_attention import GatedDeltaNet
        return GatedDeltaNet(cfg.emb_features, dtype=dtype, device=device, **cfg.mixer_options)
    if kind == "mamba2":
        from ..nn.mamba2 import Mamba2
        return Mamba2(cfg.emb_features, dtype=dtype, device=device, **cfg.mixer_options)
    if kind == "mamba":
        from ..nn.mamba import Mamba
        return Mamba(cfg.emb_features, dtype=dtype, device=device, **cfg.mixer_options)
    if kind == "kda":
        from ..nn.kda import KimiDeltaAttention
        return KimiDeltaAttention(cfg.emb_features, dtype=dtype, device=device, **cfg.mixer_options)
    if kind == "memory":
        from ..nn.memory import NeuralMemory
        return NeuralMemory(cfg.emb_features, norm_eps=cfg.norm_eps, dtype=dtype, device=device, **cfg.mixer_options)
    if kind == "mla":
        from ..nn.mla import MultiHeadLatentAttention
        return MultiHeadLatentAttention(cfg.emb_features, cfg.num_heads, norm_eps=cfg.norm_eps, dtype=dtype, device=device, **cfg.mixer_options)
    if kind == "lightning":
        from ..nn.recurrent_mixers import LightningAttention
        return LightningAttention(cfg.emb_features, layers=cfg.num_layers, norm_eps=cfg.norm_eps, dtype=dtype, device=device, **cfg.mixer_options)
    if kind == "mamba3":
        from ..nn.recurrent_mixers import Mamba3
        return Mamba3(cfg.emb_features, dtype=dtype, device=device, **cfg.mixer_options)
    if kind == "differential":
        from ..nn.attention_variants import DifferentialAttention
        return DifferentialAttention(cfg.emb_features, cfg.num_heads, cfg.num_kv_heads, layer=index, norm_eps=cfg.norm_eps, dtype=dtype, device=device)
    if kind == "forgetting":
        from ..nn.attention_variants import ForgettingAttention
        return ForgettingAttention(cfg.emb_features, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, dtype=dtype, device=device)
    if kind == "gla":
        from ..nn.linear_mixers import GatedLinearAttention
        return GatedLinearAttention(cfg.emb_features, **({"num_heads": cfg.num_heads, **cfg.mixer_options})).to(device=device, dtype=dtype)
    if kind == "delta":
        from ..nn.linear_mixers import DeltaNet
        return DeltaNet(cfg.emb_features, **({"num_heads": cfg.num_heads, **cfg.mixer_options})).to(device=device, dtype=dtype)
    if kind == "rwkv7":
        from ..nn.linear_mixers import RWKV7
        return RWKV7(cfg.emb_features, layer_index=0, **({"num_heads": cfg.num_heads, **cfg.mixer_options})).to(device=device, dtype=dtype)
    raise ValueError(f"unknown layer type {kind!r}; known: attention, local, gdn, mamba2, mamba, mamba3, kda, mla, lightning, differential, forgetting, "
                     "gla, delta, rwkv7")


class _NoNorm(nn.Module):
    """Stands where a pre-norm would: adds the pending branch into the stream and hands the stream on unnormalised."""
    weight = None

    def forward(self, h, branch=None):
        if branch is None:
            return h
        h = h + branch
        return h, h


class DecoderLayer(nn.Module):
    def __init__(self, cfg: TransformerConfig, index: int, kind: str, dtype=None, device=None):
        super().__init__()
        self.kind, self.index = kind, index
        if not cfg.pre_norm and not cfg.sandwich_norm:
            raise ValueError("a decoder without pre-norms normalises its sub-layers' outputs: set sandwich_norm=True with pre_norm=False")
        self.has_mlp = True if cfg.layer_mlp is None else bool(list(cfg.layer_mlp)[index % len(cfg.layer_mlp)])
        if kind == "none" and not self.has_mlp:
            raise ValueError(f"layer {index} has neither a mixer nor an MLP")
        if (kind == "none" or not self.has_mlp) and (cfg.sandwich_norm or not cfg.pre_norm or cfg.hyper_connections > 1 or cfg.altup > 1):
            raise NotImplementedError("layers of one sub-layer are built for the plain pre-norm block")
        self.input_norm = RMSNorm(cfg.emb_features, cfg.norm_eps, dtype=dtype, device=device) if cfg.pre_norm else _NoNorm()
        self.mixer = None if kind == "none" else _mixer(cfg, kind, dtype, device, index)
        one = kind == "none" or not self.has_mlp                  # one sub-layer: the input norm is its only norm
        self.post_norm = None if one else (RMSNorm(cfg.emb_features, cfg.norm_eps, dtype=dtype, device=device) if cfg.pre_norm else _NoNorm())
        mix = cfg.mixture
        sparse = self.has_mlp and mix is not None and (mix.layers is None or index in mix.layers)
        if not self.has_mlp:
            self.mlp = None
        elif sparse and mix.style == "clamped_glu":
            from ..nn.gpt_oss import ClampedGluMoE
            self.mlp = ClampedGluMoE(cfg.emb_features, mix, cfg.mlp_features or 4 * cfg.emb_features, init_std=cfg.init_std, dtype=dtype, device=device)
        elif sparse:
            from ..nn.moe import SparseMLP
            self.mlp = SparseMLP(cfg.emb_features, mix, cfg.mlp_features or 4 * cfg.emb_features, init_std=cfg.init_std,
                                 dtype=dtype, device=device)
        else:
            self.mlp = SwiGLU(cfg.emb_features, cfg.mlp_features or 4 * cfg.emb_features, init_std=cfg.init_std,
                              activation=cfg.mlp_activation, dtype=dtype, device=device)
        self.sparse = sparse
        self.mixer_out_norm = RMSNorm(cfg.emb_features, cfg.norm_eps, dtype=dtype, device=device) if cfg.sandwich_norm else None
        self.mlp_out_norm = RMSNorm(cfg.emb_features, cfg.norm_eps, dtype=dtype, device=device) if cfg.sandwich_norm else None
        self.tp = None          # set by parallel.tp.tensor_parallelize: branches are then partial sums over ranks
        self.cross = None       # set by the model for the layers of a loop with messages: one merge per sub-layer input
        self.residual_multiplier = float(cfg.residual_multiplier)
        self.streams = None
        if cfg.hyper_connections > 1 or cfg.altup > 1:
            from ..nn.streams import AltUp, HyperConnections
            if cfg.hyper_connections > 1:
                self.streams = nn.ModuleList([HyperConnections(cfg.emb_features, cfg.hyper_connections, 2 * index + j, dtype=dtype, device=device)
                                              for j in range(2)])
            else:
                self.streams = nn.ModuleList([AltUp(cfg.altup, 2 * index + j, device=device) for j in range(2)])

    def forward_streams(self, H, cos, sin, positions, segment_ids, cache):
        """The layer over several residual streams ``H [B,S,n,d]``: each sub-layer reads its input from the streams, and its
        output is written back by the learned connection (no fused add + norm on this path)."""
        x, ctx = self.streams[0].read(H)
        n = self.input_norm(x)
        if self.kind in ROTARY_KINDS:
            a = self.mixer(n, cos, sin, positions, segment_ids, cache, self.index)
        else:
            a = self.mixer(n, segment_ids=segment_ids, cache=cache, layer=self.index)
        H = self.streams[0].write(H, a, ctx)
        x, ctx = self.streams[1].read(H)
        return self.streams[1].write(H, self.mlp(self.post_norm(x)), ctx)

    def _norm(self, norm, h, branch):
        """Add the pending branch into the stream and normalise; under tensor parallelism the branch is a partial sum
        and the all-reduce is fused with the add and the norm."""
        if self.tp is not None and isinstance(norm, _NoNorm):
            raise NotImplementedError("tensor parallelism fuses its all-reduce with a pre-norm; a decoder without pre-norms is not built for it")
        if self.tp is not None:
            if getattr(self, "tp_training", False):
                # training: the partial sums meet in an all-reduce autograd can differentiate; the normalised activations enter
                # the next sharded product through the conjugate operator (its backward sums the partial input gradients)
                from ..parallel.tp import copy_to_region, reduce_from_region
                n, h = norm(h, reduce_from_region(branch, self.tp.group))
                return copy_to_region(n, self.tp.group), h
            return self.tp.reduce_add_norm(branch, h, norm.weight, norm.eps)
        return norm(h, branch)

    def _merged(self, h, branch, cos, sin, positions, segment_ids, bank):
        """The layer with the earlier pass's summaries merged into each sub-layer's input, before its norm."""
        h = h if branch is None else h + branch
        n = self.input_norm(self.cross[0](h, bank))
        if self.kind in ROTARY_KINDS:
            a = self.mixer(n, cos, sin, positions, segment_ids, None, self.index)
        else:
            a = self.mixer(n, segment_ids=segment_ids, cache=None, layer=self.index)
        h = h + a
        return h, self.mlp(self.post_norm(self.cross[1](h, bank)))

    def forward(self, h, branch, cos, sin, positions, segment_ids, cache, bank=None):
        """(stream, pending branch) -> (stream, pending branch); the branch is added by the next norm."""
        if bank is not None and self.cross is not None:
            return self._merged(h, branch, cos, sin, positions, segment_ids, bank)
        if branch is None:
            n = self.input_norm(h)
            if self.tp is not None and getattr(self, "tp_training", False):
                from ..parallel.tp import copy_to_region
                n = copy_to_region(n, self.tp.group)
        else:
            n, h = self._norm(self.input_norm, h, branch)
        if self.mixer is None:                                    # the MLP alone
            return h, self.mlp(n) if self.residual_multiplier == 1.0 else self.mlp(n) * self.residual_multiplier
        if self.kind in ROTARY_KINDS:
            a = self.mixer(n, cos, sin, positions, segment_ids, cache, self.index)
        else:
            a = self.mixer(n, segment_ids=segment_ids, cache=cache, layer=self.index)
        if self.mlp is None:                                      # the mixer alone
            return h, a if self.residual_multiplier == 1.0 else a * self.residual_multiplier
        if self.mixer_out_norm is not None:
            a = self.mixer_out_norm(a)
        if self.residual_multiplier != 1.0:
            a = a * self.residual_multiplier
        n, h = self._norm(self.post_norm, h, a)
        m = self.mlp(n)
        m = m if self.mlp_out_norm is None else self.mlp_out_norm(m)
        return h, (m if self.residual_multiplier == 1.0 else m * self.residual_multiplier)


class MTPBlock(nn.Module):
    """One multi-token-prediction depth (DeepSeek-V3 style): the previous depth's hidden state and the embedding of the
    next known token are normalised, concatenated, projected back to the model width and passed through one decoder
    layer; the shared head then predicts one token further ahead.  Reference: ``mtp_weight`` of
    src/dew/objectives/lm/objective.py:1348-1560 and the MTP fields of src/dew/nn/backbones/causal_transformer.py:165-423."""

    def __init__(self, cfg: TransformerConfig, index: int, dtype=None, device=None):
        super().__init__()
        self.hidden_norm = RMSNorm(cfg.emb_features, cfg.norm_eps, dtype=dtype, device=device)
        self.token_norm = RMSNorm(cfg.emb_features, cfg.norm_eps, dtype=dtype, device=device)
        self.proj = Linear(2 * cfg.emb_features, cfg.emb_features, axes=("embed", "embed"), init_std=cfg.init_std, dtype=dtype, device=device)
        self.layer = DecoderLayer(cfg, cfg.num_layers + index, "attention", dtype, device)
        self.out_norm = RMSNorm(cfg.emb_features, cfg.norm_eps, dtype=dtype, device=device)

    def forward(self, h_prev, token_emb, cos, sin, segment_ids):
        x = self.proj(torch.cat([self.hidden_norm(h_prev), self.token_norm(token_emb)], -1))
        h, branch = self.layer(x, None, cos, sin, None, segment_ids, None)
        n, _ = self.out_norm(h, branch)
        return n


@register("causal_transformer")
class CausalTransformer(nn.Module):
    def __init__(self, config: Optional[TransformerConfig] = None, dtype=None, device=None, **fields):
        super().__init__()
        cfg = config or TransformerConfig(**fields)
        self.config = cfg
        self.vocab_size = cfg.vocab_size
        self.embed = Embedding(cfg.vocab_size, cfg.emb_features, cfg.init_std, dtype=dtype, device=device)
        kinds = cfg.kinds()
        self.layers = nn.ModuleList([DecoderLayer(cfg, i, k, dtype, device) for i, k in enumerate(kinds)])
        self.final_norm = RMSNorm(cfg.emb_features, cfg.norm_eps, dtype=dtype, device=device)
        self.head = None if cfg.tie_embeddings else Linear(cfg.emb_features, cfg.vocab_size, axes=("embed", "vocab"),
                                                           init_std=cfg.init_std, dtype=dtype, device=device)
        self.mtp = nn.ModuleList([MTPBlock(cfg, i, dtype, device) for i in range(cfg.mtp_depth)]) if cfg.mtp_depth > 0 else None
        self.early_exit_gate = Linear(cfg.emb_features, 1, bias=True, init_std=cfg.init_std, dtype=dtype, device=device) \
            if cfg.loop is not None and cfg.loop.exit_gate else None
        if cfg.loop is not None and cfg.loop.messages > 0:
            if cfg.sandwich_norm or not cfg.pre_norm or cfg.layer_mlp is not None or cfg.residual_multiplier != 1.0:
                raise NotImplementedError("cross-pass messages are built for the plain pre-norm block")
            from ..nn.cross_pass import CrossPassMerge
            first, end = cfg.loop.first, cfg.num_layers if cfg.loop.end is None else cfg.loop.end
            for layer in self.layers[first:end]:
                layer.cross = nn.ModuleList(CrossPassMerge(cfg.emb_features, cfg.loop.message_rank, cfg.norm_eps, device=device) for _ in range(2))
        self.depth_sites = None
        if cfg.depth_residual_block > 0:
            if cfg.sandwich_norm or not cfg.pre_norm or cfg.loop is not None or max(cfg.hyper_connections, cfg.altup) > 1 or any(k == "none" for k in kinds):
                raise NotImplementedError("block attention residuals are built for the plain pre-norm block")
            from ..nn.depth_residuals import DepthResidualSites
            self.depth_sites = DepthResidualSites(cfg.num_layers, cfg.emb_features, cfg.norm_eps, dtype=dtype, device=device)
        self.engrams = None
        if cfg.engram:
            from ..nn.engram import Engram
            fields = {k: v for k, v in cfg.engram.items() if k != "layers"}
            self.engrams = nn.ModuleDict({str(i): Engram(cfg.emb_features, cfg.vocab_size, layer=i, norm_eps=cfg.norm_eps, dtype=dtype, device=device, **fields)
                                          for i in cfg.engram.get("layers", (0,))})
        self._rope = None

    def mtp_hiddens(self, hidden: torch.Tensor, tokens: torch.Tensor, segment_ids=None) -> List[torch.Tensor]:
        """Hidden states of the multi-token-prediction depths.  ``hidden [B,S,d]`` is the trunk's final hidden state for the
        inputs ``tokens[:, :S]``; ``tokens [B,S+1]`` carries one more token.  Depth k (1-based) returns ``[B, S-k, d]``: position
        t combines depth k-1's state at t with the embedding of token t+k and predicts token t+k+1."""
        outs = []
        cos, sin = self.rope_tables(hidden.device)
        S = hidden.shape[1]
        h = hidden
        for k, block in enumerate(self.mtp or (), start=1):
            n = S - k
            if n <= 0:
                break
            emb = self.embed(tokens[:, k:k + n])
            if self.config.embed_scale:
                emb = emb * (self.config.emb_features ** 0.5)
            seg = None if segment_ids is None else segment_ids[:, :n]
            h = block(h[:, :n], emb, cos, sin, seg)
            outs.append(h)
        return outs

    # ------------------------------------------------------------------ helpers
    def head_weight(self) -> torch.Tensor:
        return self.embed.weight if self.head is None else self.head.weight

    def rope_tables(self, device) -> Tuple[torch.Tensor, torch.Tensor]:
        cfg = self.config
        dev = torch.device(device)
        if self._rope is None or self._rope[0].device != dev:
            hd = cfg.head_dim or cfg.emb_features // cfg.num_heads
            rot = None if cfg.rotary_fraction >= 1.0 else int(hd * cfg.rotary_fraction)
            self._rope = ops.rope_tables(cfg.max_seq_len, hd, cfg.rope_theta, dev, cfg.rope_scaling, rotary_dim=rot)
        return self._rope

    def _finish(self, h, branch):
        tp = getattr(self, "tp", None)
        if tp is not None and getattr(self, "tp_training", False):
            from ..parallel.tp import reduce_from_region
            n, _ = self.final_norm(h, reduce_from_region(branch, tp.group))
        elif tp is not None:
            n, _ = tp.reduce_add_norm(branch, h, self.final_norm.weight, self.final_norm.eps)
            n = n.clone()        # the fused all-reduce returns views of a buffer later calls reuse; what leaves the model is owned
        else:
            n, _ = self.final_norm(h, branch)
        return n

    def _looped(self, h, cos, sin, positions, segment_ids, cache, train, passes: bool, steps: Optional[int]):
        """The looped trunk: returns the final-normed exit state of the last pass, or of every pass with ``passes``."""
        cfg, loop = self.config, self.config.loop
        if cache is not None:
            raise NotImplementedError("a looped decoder keeps one cache per pass; decoding with a KV cache is not built for it")
        steps = loop.steps if steps is None else steps
        first, end = loop.first, len(self.layers) if loop.end is None else loop.end
        remat = cfg.remat and train and torch.is_grad_enabled()

        def run(layers, h, branch):
            for layer in layers:
                if remat:
                    h, branch = ckpt.checkpoint(layer, h, branch, cos, sin, positions, segment_ids, None, use_reentrant=False)
                else:
                    h, branch = layer(h, branch, cos, sin, positions, segment_ids, None)
            return h, branch

        h, branch = run(self.layers[:first], h, None)
        exits = []
        if loop.messages > 0:
            if getattr(self, "tp", None) is not None:
                raise NotImplementedError("cross-pass messages are not built for tensor parallelism")
            start, bank = (h, branch), None
            looped = list(self.layers[first:end])
            for s in range(steps):
                cut = loop.backprop_steps is not None and s < steps - loop.backprop_steps and torch.is_grad_enabled()
                with torch.no_grad() if cut else contextlib.nullcontext():
                    h, branch = start
                    summaries = []
                    for j, layer in enumerate(looped):
                        if remat and not cut:
                            h, branch = ckpt.checkpoint(layer, h, branch, cos, sin, positions, segment_ids, None, bank, use_reentrant=False)
                        else:
                            h, branch = layer(h, branch, cos, sin, positions, segment_ids, None, bank)
                        if (j + 1) % loop.messages == 0 or j == len(looped) - 1:
                            summaries.append(h if branch is None else h + branch)
                    bank = torch.stack(summaries, 2)
                    if cut:
                        bank = bank.detach()
                if passes or s == steps - 1:
                    exits.append(self._finish(*run(self.layers[end:], h, branch)))
            return exits if passes else exits[-1]
        for s in range(steps):
            cut = loop.backprop_steps is not None and s < steps - loop.backprop_steps and torch.is_grad_enabled()
            if cut:
                with torch.no_grad():
                    h, branch = run(self.layers[first:end], h, branch)
                h, branch = h.detach(), (None if branch is None else branch.detach())
            else:
                h, branch = run(self.layers[first:end], h, branch)
            if passes or s == steps - 1:
                exits.append(self._finish(*run(self.layers[end:], h, branch)))
        return exits if passes else exits[-1]

    def exit_distribution(self, states: Sequence[torch.Tensor]) -> torch.Tensor:
        """``[passes, B, S]``: the probability a token exits at each pass, from the gate's hazards on the passes' exit states
        (``p_k = lambda_k prod_{j<k} (1 - lambda_j)``), the last pass taking the rest."""
        if self.early_exit_gate is None:
            raise ValueError("the model's loop has no exit gate (Loop(exit_gate=True))")
        stay = None
        out = []
        for st in states[:-1]:
            lam = torch.sigmoid(self.early_exit_gate(st).float().squeeze(-1))
            out.append(lam if stay is None else stay * lam)
            stay = (1 - lam) if stay is None else stay * (1 - lam)
        out.append(torch.ones_like(states[-1][..., 0], dtype=torch.float32) if stay is None else stay)
        return torch.stack(out)

    def hidden(self, tokens, positions=None, segment_ids=None, cache=None, train: bool = False, passes: bool = False, loop_steps: Optional[int] = None,
               embeddings: Optional[torch.Tensor] = None):
        """``embeddings [B, S, d]``: input embeddings computed by the caller (a vision-language model splices image features into the
        token embeddings); they replace the table lookup of ``tokens`` and are scaled like it."""
        cfg = self.config
        h = self.embed(tokens) if embeddings is None else embeddings
        if cfg.embed_scale:
            h = h * (cfg.emb_features ** 0.5)
        if cfg.embed_multiplier is not None:
            h = h * cfg.embed_multiplier
        cos, sin = self.rope_tables(h.device)
        n_streams = max(cfg.hyper_connections, cfg.altup)
        if n_streams > 1:
            from ..nn.streams import expand_streams
            H = expand_streams(h, n_streams)
            for layer in self.layers:
                if cfg.remat and train and torch.is_grad_enabled():
                    H = ckpt.checkpoint(layer.forward_streams, H, cos, sin, positions, segment_ids, cache, use_reentrant=False)
                else:
                    H = layer.forward_streams(H, cos, sin, positions, segment_ids, cache)
            # hyper-connections sum the streams; AltUp averages its blocks
            h = H.sum(2) if cfg.hyper_connections > 1 else H.mean(2)
            return self.final_norm(h)
        if cfg.loop is not None:
            return self._looped(h, cos, sin, positions, segment_ids, cache, train, passes, loop_steps)
        if passes:
            raise ValueError("per-pass exits need a looped decoder (TransformerConfig(loop=Loop(...)))")
        if self.depth_sites is not None:
            if getattr(self, "tp", None) is not None:
                raise NotImplementedError("block attention residuals are not built for tensor parallelism")
            from ..nn.depth_residuals import depth_residual_forward

            def call_mixer(layer, x):
                n = layer.input_norm(x)
                if layer.kind in ROTARY_KINDS:
                    return layer.mixer(n, cos, sin, positions, segment_ids, cache, layer.index)
                return layer.mixer(n, segment_ids=segment_ids, cache=cache, layer=layer.index)
            out = depth_residual_forward(self.layers, self.depth_sites, h, cfg.depth_residual_block, call_mixer,
                                         lambda layer, x: layer.mlp(layer.post_norm(x)))
            return self.final_norm(out)
        branch = None
        if self.engrams is not None and (cache is not None or tokens is None or getattr(self, "tp", None) is not None):
            raise NotImplementedError("n-gram memories read the token ids behind each position: they run on whole sequences given as tokens, without "
                                      "a KV cache and without tensor parallelism")
        for layer in self.layers:
            if self.engrams is not None and str(layer.index) in self.engrams:
                h = h if branch is None else h + branch               # the memory's gate reads the stream as the layer will see it
                h, branch = self.engrams[str(layer.index)](h, tokens, segment_ids), None
            if cfg.remat and train and torch.is_grad_enabled():
                h, branch = ckpt.checkpoint(layer, h, branch, cos, sin, positions, segment_ids, cache, use_reentrant=False)
            else:
                h, branch = layer(h, branch, cos, sin, positions, segment_ids, cache)
        return self._finish(h, branch)

    def logits(self, hidden):
        tp_head = getattr(self, "tp_head", None)
        if tp_head is not None:
            # vocabulary-parallel head: this rank's slice of the logits, gathered along the vocabulary
            local = ops.linear(hidden, tp_head)
            if self.tp.world == 1:
                return local
            parts = [torch.empty_like(local) for _ in range(self.tp.world)]
            torch.distributed.all_gather(parts, local.contiguous(), group=self.tp.group)
            return torch.cat(parts, -1)
        out = ops.linear(hidden, self.head_weight())
        if self.config.logit_divisor != 1.0:
            out = out / self.config.logit_divisor
        if self.config.logit_softcap > 0:
            out = self.config.logit_softcap * torch.tanh(out.float() / self.config.logit_softcap)
        return out

    def next_tokens_greedy(self, hidden: torch.Tensor) -> torch.Tensor:
        """argmax of the head over ``hidden [R, d]`` - under tensor parallelism without gathering the logits."""
        tp_head = getattr(self, "tp_head", None)
        if tp_head is not None and self.config.logit_softcap == 0:
            return self.tp.argmax_vocab_parallel(ops.linear(hidden, tp_head))
        return self.logits(hidden).argmax(-1)

    def forward(self, tokens, train: bool = False, decode: bool = False, positions=None, segment_ids=None, cache=None,
                return_hidden: bool = False, passes: bool = False, loop_steps: Optional[int] = None, embeddings: Optional[torch.Tensor] = None):
        h = self.hidden(tokens, positions, segment_ids, cache, train, passes, loop_steps, embeddings)
        if return_hidden:
            return h
        return [self.logits(x) for x in h] if passes else self.logits(h)

    def pop_aux(self) -> Dict[str, Any]:
        """Collect what the sparse layers recorded in the last forward: the balance loss (a metric and, when the
        objective weighs it, a loss term) and the aux-loss-free router bias updates (effects written back after the
        optimizer step; reference: ``load_balance_update`` src/dew/nn/moe.py:271)."""
        from ..nn.moe import load_balance_update
        from ..objectives.base import Ratio
        losses, effects = [], {}
        for i, layer in enumerate(self.layers):
            if not layer.sparse or not layer.mlp.last:
                continue
            last = layer.mlp.last
            losses.append(last["balance_loss"])
            bias = layer.mlp.router.expert_bias
            if bias is not None:
                effects[f"layers.{i}.mlp.router.expert_bias"] = load_balance_update(
                    bias, last["counts"], self.config.mixture.balance_rate).detach()
            layer.mlp.last = {}
        if not losses:
            return {}
        bl = torch.stack(losses).mean()
        one = torch.ones((), device=bl.device)
        return {"balance_loss": bl, "metrics": {"balance_loss": Ratio(bl.detach(), one)}, "effects": effects}

    # ------------------------------------------------------------------ accounting
    def param_count(self, active: bool = False) -> int:
        total = sum(p.numel() for p in self.parameters())
        if active and self.config.mixture is not None:
            mix = self.config.mixture
            for layer in self.layers:
                if layer.sparse:
                    per = layer.mlp.experts.param_count_per_expert()
                    total -= per * (mix.experts - mix.top_k)
        return total

    def model_flops(self, tokens: int, seq_len: int) -> float:
        """Forward FLOPs for ``tokens`` tokens in rows of ``seq_len`` (2 x params-in-matmuls x tokens + attention)."""
        cfg = self.config
        hd = cfg.head_dim or cfg.emb_features // cfg.num_heads
        # parameters that take part in a product per token: everything but the routed experts (of which a token visits
        # top_k, whatever slice of them this rank holds under expert parallelism) and the embedding table (a lookup,
        # unless it doubles as the head)
        matmul_params = 0
        for name, p in self.named_parameters():
            if ".mlp.experts." in name or name == "tp_head":
                continue
            matmul_params += p.numel()
        mix = cfg.mixture
        if mix is not None:
            sparse_layers = sum(1 for layer in self.layers if layer.sparse)
            matmul_params += sparse_layers * mix.top_k * 3 * cfg.emb_features * (mix.expert_features or cfg.mlp_features or 4 * cfg.emb_features)
        if not cfg.tie_embeddings:
            matmul_params -= self.embed.weight.numel()
        n_attn = sum(1 for k in cfg.kinds() if k in ("attention", "local"))
        attn = n_attn * 2 * 2 * cfg.num_heads * hd * seq_len / 2          # causal: half the square
        return tokens * (2.0 * matmul_params + attn)
