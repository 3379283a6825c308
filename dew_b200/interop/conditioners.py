"""Text conditioning as released text-to-image pipelines assemble it: one or several text towers (CLIP, SigLIP, T5), each with
its tokenizer, padded length and the layer its states are taken from, combined into the ``context`` (per-token states) and the
``pooled`` vector a diffusion backbone consumes.

    Stable Diffusion 1.x      one CLIP tower, last layer (after the final norm)
    SDXL                      two CLIP towers, penultimate layers concatenated along features; pooled from the second tower
    SD3 / Flux                CLIP pooled vector(s) + T5 states as the context (CLIP states zero-padded to T5's width and
                              concatenated along the sequence for SD3)

``encode`` runs without autograd in the towers' dtype; the unconditional branch of classifier-free guidance is the encoding of
the empty prompt (``negative``).

Reference: src/dew/interop/conditioners.py (binding a released pipeline's encoders), text_encoders.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.nn as nn


@dataclass
class TowerBinding:
    """One text tower of a pipeline.  ``tokenize(prompts, length) -> (ids [B, length], mask [B, length])``; ``layer``: which hidden
    state feeds the context (None: the tower's output after its final norm; -2: the penultimate block's, as SDXL takes it)."""
    tower: nn.Module
    tokenize: Callable[[Sequence[str], int], Any]
    length: int = 77
    layer: Optional[int] = None
    use_context: bool = True
    use_pooled: bool = True
    masked: bool = False                       # pass the padding mask to the tower (T5 does; CLIP pipelines do not)


class TextConditioner:
    def __init__(self, towers: Sequence[TowerBinding], combine: str = "features", context_width: Optional[int] = None):
        if combine not in ("features", "sequence"):
            raise ValueError("combine must be 'features' (concatenate widths) or 'sequence' (concatenate tokens)")
        self.towers, self.combine, self.context_width = list(towers), combine, context_width

    @torch.no_grad()
    def encode(self, prompts: Sequence[str]) -> Dict[str, torch.Tensor]:
        contexts: List[torch.Tensor] = []
        pooled: List[torch.Tensor] = []
        for b in self.towers:
            ids, mask = b.tokenize(prompts, b.length)
            dev = next(b.tower.parameters()).device
            ids, mask = ids.to(dev), (mask.to(dev) if mask is not None else None)
            km = mask if b.masked else None
            out = b.tower(ids, km) if b.layer is None else b.tower(ids, km, b.layer)
            states, vec = (out if isinstance(out, tuple) else (out, None))
            if b.use_context:
                contexts.append(states)
            if b.use_pooled and vec is not None:
                pooled.append(vec)
        result: Dict[str, torch.Tensor] = {}
        if contexts:
            if self.combine == "features":
                result["context"] = torch.cat(contexts, -1)
            else:
                width = self.context_width or max(c.shape[-1] for c in contexts)
                result["context"] = torch.cat([torch.nn.functional.pad(c, (0, width - c.shape[-1])) for c in contexts], 1)
        if pooled:
            result["pooled"] = torch.cat(pooled, -1)
        return result

    def __call__(self, prompts: Sequence[str], negative: Optional[Sequence[str]] = None) -> Dict[str, torch.Tensor]:
        """Conditional encodings, with the unconditional ones under ``uncond_*`` keys when ``negative`` is given (empty strings
        for plain classifier-free guidance)."""
        out = self.encode(prompts)
        if negative is not None:
            neg = self.encode(list(negative) if len(negative) == len(prompts) else [negative[0]] * len(prompts))
            out.update({f"uncond_{k}": v for k, v in neg.items()})
        return out


def whitespace_tokenizer(vocab_size: int, bos: int = 0, eos: int = 1, pad: Optional[int] = None):
    """A stand-in tokenizer for tests and synthetic runs: words hashed into the vocabulary, begin / end markers, padded with
    ``pad`` (default: the end marker, as CLIP pads)."""
    import zlib

    def tokenize(prompts: Sequence[str], length: int):
        ids = torch.full((len(prompts), length), eos if pad is None else pad, dtype=torch.long)
        mask = torch.zeros(len(prompts), length, dtype=torch.long)
        for i, p in enumerate(prompts):
            toks = [bos] + [2 + zlib.crc32(w.encode()) % (vocab_size - 2) for w in p.split()][: length - 2] + [eos]
            ids[i, : len(toks)] = torch.tensor(toks)
            mask[i, : len(toks)] = 1
        return ids, mask
    return tokenize
