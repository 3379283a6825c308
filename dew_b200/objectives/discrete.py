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


def entropy_bounded_choice(entropy: torch.Tensor, masked: torch.Tensor, bound: float) -> torch.Tensor:
    """Which masked places a step commits: per row, the places in order of rising entropy for as long as their entropies, less the
    largest among them, sum to at most ``bound`` - the joint error of committing them independently stays bounded, so a confident
    canvas fills in a few steps and an uncertain one a place at a time.  At least one masked place per row is always chosen.
    ``entropy, masked [R, L]`` -> boolean ``[R, L]``."""
    inf = torch.full_like(entropy, float("inf"))
    e = torch.where(masked, entropy, inf)
    order = e.argsort(-1)
    ranked = e.gather(-1, order)
    finite = torch.isfinite(ranked)
    cum = torch.where(finite, ranked, torch.zeros_like(ranked)).cumsum(-1)
    # ranked rises, so the largest entropy among the first n is the n-th
    take = finite & ((cum - ranked) <= bound)
    take[:, 0] = finite[:, 0]
    take = take.long().cummin(-1).values.bool()                 # a prefix of the ranking: nothing past the first refusal
    return torch.zeros_like(masked).scatter(-1, order, take)


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

    @torch.no_grad()
    def generate(self, variables, prompt: torch.Tensor, blocks: int, bound: float = 0.5, max_steps: Optional[int] = None, temperature: float = 0.0,
                 generator=None, stop_id: Optional[int] = None):
        """Semi-autoregressive generation: ``blocks`` new blocks after ``prompt [R, P]``, each started all-masked and refined until full.  A
        step runs the model on the prompt, the finished blocks and the current canvas, and commits the masked places
        ``entropy_bounded_choice`` picks (their argmax, or a draw at ``temperature`` > 0).  Rows that are full wait for the others; a row
        that has produced ``stop_id`` fills the rest with it.  Returns ``(tokens [R, P + blocks * block], steps [R, blocks])`` - the model
        calls each row's blocks took."""
        R, P = prompt.shape
        x = prompt
        counts = torch.zeros(R, blocks, dtype=torch.long)
        limit = max_steps or self.block
        done = torch.zeros(R, dtype=torch.bool, device=prompt.device)
        for b in range(blocks):
            canvas = torch.full((R, self.block), self.mask_id, dtype=torch.long, device=prompt.device)
            if stop_id is not None:
                canvas = torch.where(done[:, None], torch.full_like(canvas, stop_id), canvas)
            for it in range(limit):
                masked = canvas == self.mask_id
                if not bool(masked.any()):
                    break
                logits = self.apply(variables, torch.cat([x, canvas], 1))
                logits = (logits[0] if isinstance(logits, tuple) else logits)[:, -self.block:].float()
                logits[..., self.mask_id] = -float("inf")
                logp = torch.log_softmax(logits, -1)
                entropy = -(logp.exp() * logp.clamp_min(-1e30)).sum(-1)
                if temperature > 0:
                    draw = torch.multinomial((logits / temperature).softmax(-1).reshape(-1, logits.shape[-1]), 1, generator=generator).view(R, self.block)
                else:
                    draw = logits.argmax(-1)
                last = it == limit - 1
                choose = masked if last else entropy_bounded_choice(entropy, masked, bound)
                canvas = torch.where(choose, draw, canvas)
                counts[:, b] += masked.any(-1).long().cpu()
            if stop_id is not None:
                hit = (canvas == stop_id)
                after = hit.long().cumsum(-1) > 0
                canvas = torch.where(after, torch.full_like(canvas, stop_id), canvas)
                done = done | hit.any(-1)
            x = torch.cat([x, canvas], 1)
        return x, counts
