"""How a run trains its routers: one policy that any objective composes with its own loss.

``ExpertBalance`` holds up to three optional terms: the aux-loss-free balancing bias (``balance_rate``, arXiv 2408.15664),
DeepSeek-V2's expert-level balance loss (``aux_loss_alpha``, per sequence with ``seq_aux``) and ST-MoE's router z-loss
(``router_z_loss``, arXiv 2202.08906).  The sparse layers record what their router saw in the last forward
(``MoE.last``: scores, chosen experts, log partition); ``compose`` reads those records, adds the loss terms to the
objective's statistic and returns the bias updates as effects, which the trainer writes back once per committed update.

Reference: src/dew/objectives/routing.py (``ExpertBalance`` :74-243, ``refuse_fixed_routers`` :249, ``router_counts`` :319,
``router_z_terms`` :348, ``router_moments`` :370).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Iterator, Optional, Tuple

import torch

from .base import Aux, Ratio


class UntrainedRouter(ValueError):
    """A router that nothing trains: no gradient reaches it and no bias update moves it."""


def sparse_layers(model: torch.nn.Module) -> Iterator[Tuple[str, Any]]:
    """(module path, MoE layer) for every sparse layer of ``model``."""
    from ..nn.moe import SparseMLP as MoE
    for name, module in model.named_modules():
        if isinstance(module, MoE):
            yield name, module


def router_balance_loss(scores: torch.Tensor, ids: torch.Tensor, experts: int, sequences: Optional[torch.Tensor] = None) -> torch.Tensor:
    """DeepSeek-V2's expert-level balance loss ``sum_i f_i P_i`` with ``f_i = E / (K T) * #{tokens choosing i}`` and ``P_i`` the
    mean normalised score of expert i.  ``sequences [T]`` (ids, -1 = padding) gives the per-sequence form: the loss of each
    sequence alone, averaged over the sequences."""
    T, K = ids.shape
    norm = scores / scores.sum(-1, keepdim=True).clamp_min(1e-20)
    chosen = torch.zeros(T, experts, device=ids.device, dtype=torch.float32).scatter_add_(1, ids, torch.ones_like(ids, dtype=torch.float32))
    if sequences is None:
        f = chosen.sum(0) * (experts / (K * T))
        return (f * norm.mean(0)).sum()
    valid = sequences >= 0
    uniq, inverse = torch.unique(sequences[valid], return_inverse=True)
    S = uniq.numel()
    counts = torch.zeros(S, device=ids.device).index_add_(0, inverse, torch.ones_like(inverse, dtype=torch.float32))
    f = torch.zeros(S, experts, device=ids.device).index_add_(0, inverse, chosen[valid]) * (experts / (K * counts[:, None]))
    P = torch.zeros(S, experts, device=ids.device).index_add_(0, inverse, norm[valid]) / counts[:, None]
    return (f * P).sum(-1).mean()


@dataclass(frozen=True)
class ExpertBalance:
    """``balance_rate``: step of the selection-only bias against each expert's load, per committed update (None leaves the
    bias alone; the mixture must keep one, ``bias=True``).  ``aux_loss_alpha``: weight of the balance loss summed over the
    routers (``seq_aux``: each sequence of a row balanced alone).  ``router_z_loss``: weight of the mean squared log partition
    of every router's logits, summed over the routers."""
    balance_rate: Optional[float] = None
    aux_loss_alpha: Optional[float] = None
    seq_aux: bool = True
    router_z_loss: float = 0.0

    def __post_init__(self):
        if self.balance_rate is not None and not (0 < self.balance_rate < math.inf):
            raise ValueError(f"balance_rate moves each bias by this much per update, so it is positive and finite, got {self.balance_rate}")
        if self.aux_loss_alpha is not None and not (0 < self.aux_loss_alpha < math.inf):
            raise ValueError(f"aux_loss_alpha scales the balance loss, so it is positive and finite, got {self.aux_loss_alpha}")
        if not (0 <= self.router_z_loss < math.inf):
            raise ValueError(f"router_z_loss is finite and nonnegative, got {self.router_z_loss}")

    def prepare(self, model: torch.nn.Module) -> None:
        """Ask the sparse layers to keep what the terms read (scores and choices per token, log partitions)."""
        found = False
        for _, layer in sparse_layers(model):
            found = True
            layer.keep_router_outputs = self.aux_loss_alpha is not None or self.router_z_loss > 0
            if self.balance_rate is not None and layer.router.expert_bias is None:
                raise UntrainedRouter("balance_rate moves the routers' balancing bias, and this mixture keeps none (bias=False)")
        if not found:
            raise ValueError("the model has no sparse layer, so there is no router to balance")

    def compose(self, model: torch.nn.Module, prediction: Ratio, sequences: Optional[torch.Tensor] = None) -> Tuple[Ratio, Aux]:
        """``prediction`` plus the router terms (each weighted by the prediction's mass, so the pooled mean adds them once),
        with metrics and the bias updates as effects.  ``sequences [B, S]``: document ids of a packed batch (or None: every row
        is one sequence)."""
        from ..nn.moe import load_balance_update
        total, mass = prediction.total, prediction.mass
        balance, z, effects, n = 0.0, 0.0, {}, 0
        for name, layer in sparse_layers(model):
            last = layer.last
            if not last:
                continue
            n += 1
            E = layer.mix.experts
            if self.aux_loss_alpha is not None:
                seq = None
                if self.seq_aux:
                    B, S = last["shape"]
                    rows = torch.arange(B, device=last["ids"].device)[:, None].expand(B, S)
                    if sequences is not None:
                        seq = torch.where(sequences >= 0, rows * (int(sequences.max()) + 1) + sequences.clamp_min(0), torch.full_like(rows, -1))
                    else:
                        seq = rows
                    seq = seq.reshape(-1)
                balance = balance + router_balance_loss(last["scores"], last["ids"], E, seq)
            if self.router_z_loss > 0:
                z = z + last["log_z"].pow(2).mean()
            if self.balance_rate is not None and layer.router.expert_bias is not None:
                effects[f"{name}.router.expert_bias"] = load_balance_update(layer.router.expert_bias, last["counts"], self.balance_rate).detach()
            layer.last = {}
        metrics: Dict[str, Any] = {}
        one = torch.ones((), device=mass.device)
        if self.aux_loss_alpha is not None and n:
            total = total + self.aux_loss_alpha * balance * mass
            metrics["router_balance_loss"] = Ratio(balance.detach(), one)
        if self.router_z_loss > 0 and n:
            total = total + self.router_z_loss * z * mass
            metrics["router_z_loss"] = Ratio(z.detach(), one)
        return Ratio(total, mass), Aux(metrics=metrics, effects=effects)


def refuse_fixed_routers(model: torch.nn.Module, balance: Optional[ExpertBalance]) -> None:
    """Raise ``UntrainedRouter`` when a router of ``model`` would stay where it starts: its weight takes no gradient
    (``requires_grad`` off) and no bias update moves its selection."""
    for name, layer in sparse_layers(model):
        trained = layer.router.weight.requires_grad
        biased = balance is not None and balance.balance_rate is not None and layer.router.expert_bias is not None
        if not trained and not biased:
            raise UntrainedRouter(f"the router of {name!r} is frozen and no balance_rate moves its bias: nothing trains it")
