"""Discrete (masked) diffusion language models.

``MaskedDiffusionLM`` (MDLM): a token is masked with probability ``t ~ U(eps, 1)`` per row; the model (bidirectional
attention, no causal mask) predicts the clean tokens at the masked positions; the negative ELBO weights the masked
cross-entropy by ``1 / t`` (the log-linear schedule).  ``BlockDiffusionLM`` masks inside blocks only, conditioning every
block on the clean blocks before it (block-causal attention is the model's business; the objective supplies the mask and
weights).  ``sample`` runs the ancestral unmasking schedule.

Reference: src/dew/diffusion/discrete.py (716 lines, MDLM), src/dew/diffusion/block.py (446),
src/dew/objectives/diffusion/{masked,block}.py, examples/train_masked_lm.py.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .base import Aux, Objective, Ratio, Step


class MaskedDiffusionLM(Objective):
    def __init__(self, model, mask_id: int, eps: float = 1e-3, ema_decay: Optional[float] = None, pad_id: Optional[int] = None):
        self.model, self.mask_id, self.eps, self.ema_decay, self.pad_id = model, mask_id, eps, ema_decay, pad_id

    def corrupt(self, tokens: torch.Tensor, step: Step):
        rows, T = tokens.shape
        t = self.eps + (1 - self.eps) * step.sample("mask_rate", (1,), rows, kind="uniform").to(tokens.device)      # [rows, 1]
        u = step.sample("mask_draw", (T,), rows, kind="uniform").to(tokens.device)
        masked = u < t
        if self.pad_id is not None:
            masked &= tokens != self.pad_id
        return torch.where(masked, torch.full_like(tokens, self.mask_id), tokens), masked, t

    def loss(self, variables, batch, step: Step):
        tokens = batch["tokens"]
        noisy, masked, t = self.corrupt(tokens, step)
        logits = self.apply(variables, noisy).float()
        ce = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), tokens.reshape(-1), reduction="none").view_as(tokens)
        weighted = (ce * masked.float() / t).sum()
        mass = torch.tensor(float(tokens.numel() if self.pad_id is None else int((tokens != self.pad_id).sum())), device=ce.device)
        acc = Ratio(((logits.argmax(-1) == tokens) & masked).sum().float(), masked.sum().float().clamp_min(1))
        return Ratio(weighted, mass), Aux(metrics={"masked_accuracy": acc, "masked_ce": Ratio((ce * masked).sum(), masked.sum().float().clamp_min(1))})

    @torch.no_grad()
    def sample(self, variables, rows: int, length: int, steps: int = 16, generator=None, device="cpu", temperature: float = 1.0):
        """Ancestral unmasking: start all-masked; at step i a masked position is revealed with probability
        ``(t_i - t_{i+1}) / t_i`` and takes a draw from the model's categorical; the last step reveals the rest."""
        x = torch.full((rows, length), self.mask_id, dtype=torch.long, device=device)
        ts = torch.linspace(1.0, 0.0, steps + 1)
        for i in range(steps):
            logits = self.apply(variables, x).float() / max(temperature, 1e-6)
            logits[..., self.mask_id] = -float("inf")
            draw = torch.multinomial(logits.softmax(-1).reshape(-1, logits.shape[-1]), 1, generator=generator).view(rows, length)
            p = 1.0 if i == steps - 1 else float((ts[i] - ts[i + 1]) / ts[i])
            reveal = (x == self.mask_id) & (torch.rand(rows, length, generator=generator, device="cpu").to(device) < p)
            x = torch.where(reveal, draw, x)
        return x


class BlockDiffusionLM(MaskedDiffusionLM):
    """Masked diffusion inside blocks of ``block`` tokens; each row draws one rate per block (so blocks sit at different
    noise levels, as in semi-autoregressive sampling) and the model is expected to attend block-causally."""

    def __init__(self, model, mask_id: int, block: int = 16, **kw):
        super().__init__(model, mask_id, **kw)
        self.block = block

    def corrupt(self, tokens, step: Step):
        rows, T = tokens.shape
        nb = (T + self.block - 1) // self.block
        tb = self.eps + (1 - self.eps) * step.sample("block_rate", (nb,), rows, kind="uniform").to(tokens.device)
        t = tb.repeat_interleave(self.block, 1)[:, :T]
        u = step.sample("mask_draw", (T,), rows, kind="uniform").to(tokens.device)
        masked = u < t
        if self.pad_id is not None:
            masked &= tokens != self.pad_id
        return torch.where(masked, torch.full_like(tokens, self.mask_id), tokens), masked, t

    @staticmethod
    def block_causal_mask(T: int, block: int, device="cpu") -> torch.Tensor:
        """``[T, T]`` boolean: position i may attend to j when j's block is not later than i's."""
        b = torch.arange(T, device=device) // block
        return b[:, None] >= b[None, :]
