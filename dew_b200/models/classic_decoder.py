"""The decoder lineage before RMSNorm and gated MLPs: biased LayerNorm, a two-matrix MLP, learned / rotary / ALiBi positions, and the
three block shapes its families use - sequential pre-norm (GPT-2, OPT, BLOOM, StarCoder2, GPTBigCode), parallel with one norm
(Falcon-7B, Phi) or two (GPT-NeoX), and post-norm (GPT-1, OPT-350m).  One ``ClassicConfig`` says which; ``interop/classic.py`` reads the
published checkpoints of those families into it.

The projections run through the library's ``Linear`` (the tcgen05 GEMM on a GPU) and attention through ``ops.attention`` unless a
bias (ALiBi) forces the score-matrix form.  Generation keeps plain per-layer key / value tensors (``ClassicCache``): these families
are loaded to be evaluated, distilled from or fine-tuned, not served at scale - the paged server belongs to ``CausalTransformer``.

Reference: src/dew/interop/families/gpt2.py, gpt_neox.py, falcon.py, phi.py, opt.py, bloom.py, starcoder2.py, gpt_bigcode.py (the blocks
those families translate into), src/dew/interop/decoder_parts.py.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..nn.layers import Embedding, LayerNorm, Linear

ACTIVATIONS = {
    "gelu": lambda x: F.gelu(x),
    "gelu_tanh": lambda x: F.gelu(x, approximate="tanh"),
    "relu": F.relu,
    "silu": F.silu,
}


@dataclass
class ClassicConfig:
    vocab_size: int = 50257
    emb_features: int = 768
    num_layers: int = 12
    num_heads: int = 12
    num_kv_heads: Optional[int] = None                # 1: multi-query (Falcon-7B, GPTBigCode)
    mlp_features: Optional[int] = None                # 4 x emb_features by default
    max_seq_len: int = 1024
    positions: str = "learned"                        # learned | rotary | alibi
    position_offset: int = 0                          # OPT: its position table starts at row 2
    rope_theta: float = 10000.0
    rotary_fraction: float = 1.0                      # share of a head that rotates; heads laid out [rotated a | kept a | rotated b | kept b]
    norm_eps: float = 1e-5
    activation: str = "gelu_tanh"
    block: str = "sequential"                         # sequential | parallel | post_norm
    parallel_norms: int = 1                           # parallel block: 1 - both branches read one norm; 2 - each its own
    attn_bias: bool = True                            # on q | k | v and on the output projection
    mlp_bias: bool = True
    embed_norm: bool = False                          # BLOOM: LayerNorm on the embeddings
    final_norm: bool = True                           # (a post-norm stack ends normalised already)
    embed_proj: Optional[int] = None                  # OPT-350m: the embedding at a width of its own, projected in and out
    tie_embeddings: bool = True
    head_bias: bool = False                           # Phi
    window: Optional[int] = None                      # StarCoder2
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.emb_features // self.num_heads


def alibi_slopes(heads: int) -> torch.Tensor:
    """Per-head slopes: a geometric sequence starting at ``2 ** (-8 / n)`` for the largest power of two ``n <= heads``; further heads take
    every other term of the sequence for ``2 n``."""
    n = 2 ** math.floor(math.log2(heads))
    base = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
    slopes = [base ** (i + 1) for i in range(n)]
    if n < heads:
        extra = 2.0 ** (-(2.0 ** -(math.log2(2 * n) - 3)))
        slopes += [extra ** (2 * i + 1) for i in range(heads - n)]
    return torch.tensor(slopes, dtype=torch.float32)


class ClassicCache:
    """Per layer, the keys and values seen so far, ``[B, T, Hkv, D]``."""

    def __init__(self, layers: int):
        self.k: List[Optional[torch.Tensor]] = [None] * layers
        self.v: List[Optional[torch.Tensor]] = [None] * layers

    @property
    def length(self) -> int:
        return 0 if self.k[0] is None else int(self.k[0].shape[1])

    def extend(self, layer: int, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.k[layer] is not None:
            k, v = torch.cat([self.k[layer], k], 1), torch.cat([self.v[layer], v], 1)
        self.k[layer], self.v[layer] = k, v
        return k, v


class ClassicBlock(nn.Module):
    def __init__(self, cfg: ClassicConfig, index: int, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        E, H, Hkv, D = cfg.emb_features, cfg.num_heads, cfg.num_kv_heads or cfg.num_heads, cfg.head_dim
        self.cfg, self.index, self.H, self.Hkv, self.D = cfg, index, H, Hkv, D
        self.norm1 = LayerNorm(E, cfg.norm_eps, **kw)
        self.norm2 = LayerNorm(E, cfg.norm_eps, **kw) if not (cfg.block == "parallel" and cfg.parallel_norms == 1) else None
        self.qkv = Linear(E, (H + 2 * Hkv) * D, bias=cfg.attn_bias, axes=("embed", "heads"), init_std=cfg.init_std, **kw)
        self.out = Linear(H * D, E, bias=cfg.attn_bias, axes=("heads", "embed"), init_std=cfg.init_std / math.sqrt(2 * cfg.num_layers), **kw)
        Fw = cfg.mlp_features or 4 * E
        self.fc1 = Linear(E, Fw, bias=cfg.mlp_bias, init_std=cfg.init_std, **kw)
        self.fc2 = Linear(Fw, E, bias=cfg.mlp_bias, axes=("mlp", "embed"), init_std=cfg.init_std / math.sqrt(2 * cfg.num_layers), **kw)
        self.act = ACTIVATIONS[cfg.activation]

    def attend(self, x, cos, sin, positions, slopes, cache: Optional[ClassicCache]):
        B, S, _ = x.shape
        H, Hkv, D = self.H, self.Hkv, self.D
        qkv = self.qkv(x).view(B, S, H + 2 * Hkv, D)
        if cos is not None:
            qkv = ops.rope(qkv, cos, sin, positions, rot_heads=H + Hkv)
        q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
        if cache is not None:
            k, v = cache.extend(self.index, k, v)
        T = k.shape[1]
        if slopes is None and (cache is None or S == T):
            o = ops.attention(q, k, v, causal=True, window=self.cfg.window)
        else:
            # the score-matrix form: ALiBi's per-head linear bias over key positions, or a query block against a longer cache
            from ..nn.attention_variants import biased_attention
            qi = torch.arange(T - S, T, device=x.device)[:, None]
            ki = torch.arange(T, device=x.device)[None, :]
            mask = ki <= qi
            if self.cfg.window:
                mask = mask & (ki > qi - self.cfg.window)
            bias = None if slopes is None else (slopes.to(x.device)[:, None, None] * (ki - qi)[None].float())[None]
            o = biased_attention(q, k, v, bias=bias, mask=mask[None, None])
        return self.out(o.reshape(B, S, H * D))

    def mlp(self, x):
        return self.fc2(self.act(self.fc1(x)))

    def forward(self, x, cos, sin, positions, slopes, cache):
        kind = self.cfg.block
        if kind == "parallel":
            n = self.norm1(x)
            return x + self.attend(n, cos, sin, positions, slopes, cache) + self.mlp(n if self.norm2 is None else self.norm2(x))
        if kind == "post_norm":
            x = self.norm1(x + self.attend(x, cos, sin, positions, slopes, cache))
            return self.norm2(x + self.mlp(x))
        x = x + self.attend(self.norm1(x), cos, sin, positions, slopes, cache)
        return x + self.mlp(self.norm2(x))


class ClassicDecoder(nn.Module):
    def __init__(self, config: Optional[ClassicConfig] = None, dtype=None, device=None, **fields):
        super().__init__()
        cfg = config if config is not None else ClassicConfig(**fields)
        if cfg.positions not in ("learned", "rotary", "alibi") or cfg.block not in ("sequential", "parallel", "post_norm"):
            raise ValueError(f"positions {cfg.positions!r} / block {cfg.block!r}: known positions learned | rotary | alibi, blocks sequential | parallel | post_norm")
        self.config = cfg
        kw = dict(dtype=dtype, device=device)
        Ew = cfg.embed_proj or cfg.emb_features
        self.embed = Embedding(cfg.vocab_size, Ew, cfg.init_std, **kw)
        self.positions = Embedding(cfg.max_seq_len + cfg.position_offset, cfg.emb_features, cfg.init_std, **kw) if cfg.positions == "learned" else None
        self.project_in = Linear(Ew, cfg.emb_features, **kw) if cfg.embed_proj else None
        self.project_out = Linear(cfg.emb_features, Ew, **kw) if cfg.embed_proj else None
        self.embed_norm = LayerNorm(cfg.emb_features, cfg.norm_eps, **kw) if cfg.embed_norm else None
        self.layers = nn.ModuleList(ClassicBlock(cfg, i, **kw) for i in range(cfg.num_layers))
        self.final_norm = LayerNorm(cfg.emb_features, cfg.norm_eps, **kw) if cfg.final_norm else None
        self.head = None if cfg.tie_embeddings else Linear(Ew, cfg.vocab_size, bias=cfg.head_bias, axes=("embed", "vocab"), init_std=cfg.init_std, **kw)
        self._rope = None
        self._slopes = alibi_slopes(cfg.num_heads) if cfg.positions == "alibi" else None

    @property
    def head_parameter(self) -> torch.Tensor:
        return self.embed.weight if self.head is None else self.head.weight

    def rope_tables(self, device):
        cfg = self.config
        if cfg.positions != "rotary":
            return None, None
        if self._rope is None or self._rope[0].device != torch.device(device):
            rot = None if cfg.rotary_fraction >= 1.0 else int(cfg.head_dim * cfg.rotary_fraction)
            self._rope = ops.rope_tables(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta, device, None, rotary_dim=rot)
        return self._rope

    def hidden(self, tokens, positions=None, cache: Optional[ClassicCache] = None):
        cfg = self.config
        B, S = tokens.shape
        if positions is None:
            start = cache.length if cache is not None else 0
            positions = torch.arange(start, start + S, device=tokens.device)[None].expand(B, S)
        h = self.embed(tokens)
        if self.project_in is not None:
            h = self.project_in(h)
        if self.positions is not None:
            h = h + self.positions(positions + cfg.position_offset)
        if self.embed_norm is not None:
            h = self.embed_norm(h)
        cos, sin = self.rope_tables(h.device)
        for layer in self.layers:
            h = layer(h, cos, sin, positions if cos is not None else None, self._slopes, cache)
        if self.final_norm is not None:
            h = self.final_norm(h)
        return h if self.project_out is None else self.project_out(h)

    def logits(self, hidden):
        if self.head is None:
            return ops.linear(hidden, self.embed.weight)
        return self.head(hidden)

    def forward(self, tokens, positions=None, cache: Optional[ClassicCache] = None):
        return self.logits(self.hidden(tokens, positions, cache))

    def new_cache(self) -> ClassicCache:
        return ClassicCache(self.config.num_layers)

    @torch.no_grad()
    def generate(self, tokens: torch.Tensor, new_tokens: int, temperature: float = 0.0, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """Greedy (``temperature`` 0) or sampled continuation of ``tokens [B, S]`` with the per-layer cache."""
        cache = self.new_cache()
        logits = self(tokens, cache=cache)[:, -1]
        out = [tokens]
        for _ in range(new_tokens):
            if temperature > 0:
                nxt = torch.multinomial(torch.softmax(logits.float() / temperature, -1), 1, generator=generator)
            else:
                nxt = logits.argmax(-1, keepdim=True)
            out.append(nxt)
            logits = self(nxt, cache=cache)[:, -1]
        return torch.cat(out, 1)
