"""Training without backpropagation: node perturbation for a language model.

Every dense / embedding layer's output is jittered by ``sigma * eps`` (``eps`` standard normal) in an antithetic pair of
forward passes; each token is credited by its own loss difference ``c = (l+ - l-) / (2 sigma)``, and ``c * eps`` estimates the
loss's gradient at that layer's output for that token.  The layer's weight gradient then follows locally (for ``y = x W^T``:
``sum_t (c_t eps_t) x_t^T``), with nothing propagated between layers.  ``draws`` pairs are averaged per step.

The objective returns the clean loss as its value and a surrogate's gradient: a third pass computes every perturbed layer
from a detached input, and ``sum <y, stopgrad(c * eps)>`` is added with zero value, so the trainer's ordinary backward
produces the estimates (and only them: no gradient crosses a layer boundary).

Reference: src/dew/objectives/perturbation.py (``NodePerturbation``), examples/forward_only_lm.py.
"""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..utils import keys as K
from .base import Aux, Objective, Ratio, Step


def _perturbed(model: nn.Module) -> List[nn.Module]:
    from ..nn.layers import Embedding, Linear
    return [m for m in model.modules() if isinstance(m, (Linear, Embedding, nn.Linear, nn.Embedding))]


class NodePerturbation(Objective):
    def __init__(self, model: nn.Module, seq_len: int, sigma: float = 1e-2, draws: int = 1, ema_decay=None, pad_id=None):
        if sigma <= 0 or draws < 1:
            raise ValueError("node perturbation needs sigma > 0 and at least one draw")
        self.model, self.seq_len, self.sigma, self.draws, self.ema_decay, self.pad_id = model, seq_len, float(sigma), int(draws), ema_decay, pad_id
        self.nodes = _perturbed(model)
        if not self.nodes:
            raise ValueError("the model has no dense or embedding layer to perturb")

    def _token_losses(self, variables, tokens, head=None):
        """Per-token losses.  ``head(hidden) -> logits`` replaces the model's own head call when the head is a bare weight
        (no module whose output a hook could reach): it is then perturbed and credited as one more node."""
        if head is not None and hasattr(self.model, "logits"):
            logits = head(self.apply(variables, tokens[:, :-1], return_hidden=True)).float()
        else:
            logits = self.apply(variables, tokens[:, :-1]).float()
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), tokens[:, 1:].reshape(-1), reduction="none").view(tokens.shape[0], -1)

    def loss(self, variables, batch, step: Step):
        tokens = batch["tokens"]
        B, S = tokens.shape[0], tokens.shape[1] - 1
        weight = torch.ones(B, S, device=tokens.device) if self.pad_id is None else (tokens[:, 1:] != self.pad_id).float()
        mass = weight.sum()
        if not step.train:
            with torch.no_grad():
                clean = self._token_losses(variables, tokens)
            return Ratio((clean * weight).sum(), mass), Aux()
        noise: Dict[int, torch.Tensor] = {}
        credit: Dict[int, torch.Tensor] = {}
        sign = [1.0]
        gen = K.generator(step.fold("node perturbation")) if hasattr(step, "fold") else torch.Generator().manual_seed(0)

        def jitter(index):
            def hook(module, args, out):
                if index not in noise:
                    noise[index] = torch.randn(out.shape, generator=gen).to(out.device, out.dtype)
                return out + (sign[0] * self.sigma) * noise[index]
            return hook
        HEAD = -1

        def noisy_head(hidden):
            out = self.model.logits(hidden)
            if HEAD not in noise:
                noise[HEAD] = torch.randn(out.shape, generator=gen).to(out.device, out.dtype)
            return out + (sign[0] * self.sigma) * noise[HEAD]
        own_head = noisy_head if hasattr(self.model, "logits") else None
        for _ in range(self.draws):
            noise.clear()
            handles = [m.register_forward_hook(jitter(i)) for i, m in enumerate(self.nodes)]
            try:
                with torch.no_grad():
                    sign[0] = 1.0
                    plus = self._token_losses(variables, tokens, own_head)
                    sign[0] = -1.0
                    minus = self._token_losses(variables, tokens, own_head)
            finally:
                for h in handles:
                    h.remove()
            c = ((plus - minus) / (2 * self.sigma) * weight)                         # [B, S]: each token's own credit
            for i, eps in noise.items():
                cc = c.reshape(B, S, *([1] * (eps.dim() - 2))) if eps.dim() >= 2 and eps.shape[:2] == (B, S) else c.mean()
                credit[i] = credit.get(i, 0) + (cc * eps.float()) / self.draws
        # the local pass: every perturbed layer reads a detached input; <y, credit> carries the estimates into backward
        surrogate = [torch.zeros((), device=tokens.device)]

        def cut(module, args):
            return tuple(a.detach() if torch.is_tensor(a) and a.is_floating_point() else a for a in args)

        def collect(index):
            def hook(module, args, out):
                surrogate[0] = surrogate[0] + (out.float() * credit[index].to(out.device)).sum()
            return hook
        handles = [m.register_forward_pre_hook(cut) for m in self.nodes] + [m.register_forward_hook(collect(i)) for i, m in enumerate(self.nodes)]
        def local_head(hidden):
            out = self.model.logits(hidden.detach())
            surrogate[0] = surrogate[0] + (out.float() * credit[HEAD].to(out.device)).sum()
            return out
        try:
            clean = self._token_losses(variables, tokens, local_head if own_head is not None else None)
        finally:
            for h in handles:
                h.remove()
        value = (clean.detach() * weight).sum()
        total = value + (surrogate[0] - surrogate[0].detach())
        return Ratio(total, mass), Aux(metrics={"credit_abs": Ratio(c.abs().sum().detach(), mass)})
