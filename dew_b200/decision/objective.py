"""``DecisionObjective``: training a decision model on labelled questions.

``batch(examples)`` lays the examples out (``Layout.rows``), packs the rows first-fit into windows of one length and returns a
dict of tensors (the ``DecisionInputs`` fields plus ``targets [B, Q, K]``, ``scored [B, Q]``, ``weights [B, Q]`` and the consistency
groups), whose leading dimension a trainer may split into microbatches.  ``loss`` charges every scored question by a proper
scoring rule against its gold distribution, smoothed by ``smoothing`` over the question's own options, and pools exactly
(``Ratio(sum of weighted charges, sum of weights)``).  With ``consistency > 0`` the questions of a group (the same question
negated, paraphrased, its options re-ordered) are also held to one answer: each member's distribution is carried onto the
group's canonical keys and charged its divergence from the members' mean (a generalised Jensen-Shannon term).

Reference: src/dew/decision/objective.py (``DecisionObjective``: scoring rule, smoothing, ``consistency``, ``evaluate`` ->
``Decisions``), src/dew/decision/rows.py.
"""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..objectives.base import Aux, Objective, Ratio, Step
from .data import Example, Group, GroupedExamples
from .inputs import DecisionInputs, collate, first_fit
from .layout import Layout, Refused
from .metrics import Decisions
from .model import DecisionModel
from .scoring import LogLoss, ScoringRule, probabilities, rule_named


def _question_id(q) -> int:
    return hash(q) & 0x7FFFFFFFFFFF


class DecisionObjective(Objective):
    def __init__(self, model: DecisionModel, layout: Layout, rule: Union[str, ScoringRule] = "log", smoothing: float = 0.0,
                 consistency: float = 0.0, length: Optional[int] = None, questions: Optional[int] = None, options: Optional[int] = None,
                 ema_decay: Optional[float] = None, skip_refused: bool = True):
        if not 0.0 <= smoothing < 1.0:
            raise ValueError("label smoothing lies in [0, 1)")
        self.model, self.layout = model, layout
        self.rule = rule_named(rule) if isinstance(rule, str) else rule
        self.smoothing, self.consistency = float(smoothing), float(consistency)
        self.length = length or layout.max_len
        self.questions, self.options = questions, options
        self.ema_decay = ema_decay
        self.skip_refused = skip_refused
        self.refused: Dict[str, int] = {}

    # ------------------------------------------------------------------ examples -> tensors
    def batch(self, examples: Sequence[Union[Example, GroupedExamples]], windows: Optional[int] = None) -> Dict[str, torch.Tensor]:
        rows, golds, weights, ids, members = [], [], [], [], []
        groups: List[Tuple[Group, Dict[str, int]]] = []          # (group, member key -> flat question index)
        flat = 0
        for ex in examples:
            units = [(None, ex)] if isinstance(ex, Example) else list(enumerate(ex.examples))
            local: Dict[str, int] = {}
            for idx, e in units:
                try:
                    laid = self.layout.rows(e.state, e.questions)
                except Refused as r:
                    if not self.skip_refused:
                        raise
                    self.refused[r.reason] = self.refused.get(r.reason, 0) + 1
                    continue
                for r in laid:
                    rows.append(r)
                    for name in r.names:
                        golds.append(e.distribution(name))
                        weights.append(e.weight)
                        ids.append(_question_id(e.questions[name]))
                        local[name if idx is None else f"{idx}.{name}"] = flat
                        members.append((e, name))
                        flat += 1
                if idx is None:
                    groups += [(g, local) for g in e.groups]
            if not isinstance(ex, Example):
                groups += [(g, local) for g in ex.groups]
        if not rows:
            raise ValueError("no example of the batch could be laid out")
        Q = self.questions or max(len(r.names) for r in rows)
        K = self.options or max(max(r.counts) for r in rows)
        placed, leftover = first_fit(rows, self.length, windows, None)
        if leftover:
            raise ValueError(f"{len(leftover)} rows found no room in {windows} windows of {self.length} tokens")
        Q = max(Q, max(sum(len(rows[i].names) for i in w) for w in placed))
        inputs, where = collate(rows, placed, self.length, Q, K, self.layout.specials.pad, batch=windows)
        B = inputs.tokens.shape[0]
        targets = torch.zeros(B, Q, K)
        scored = torch.zeros(B, Q, dtype=torch.bool)
        weight = torch.zeros(B, Q)
        classes = torch.zeros(B, Q, dtype=torch.int64)
        slot_of: List[Tuple[int, int]] = [s for w in where for s in w]
        for f, (b, q) in enumerate(slot_of):
            classes[b, q] = ids[f]
            if golds[f] is not None:
                targets[b, q, : len(golds[f])] = torch.tensor(golds[f], dtype=torch.float32)
                scored[b, q] = True
                weight[b, q] = weights[f]
        out = {**inputs.as_batch(), "targets": targets, "scored": scored, "weights": weight, "classes": classes}
        # consistency groups: a group id per question slot and, per option, its canonical index
        group_id = torch.zeros(B, Q, dtype=torch.int64)
        canon = torch.zeros(B, Q, K, dtype=torch.int64)
        gid = 0
        for g, local in groups:
            if not all(m in local for m in g.members):
                continue                                                # a member's row was refused: the group is not held
            gid += 1
            keys = g.canonical()
            for m, mapping in g.members.items():
                b, q = slot_of[local[m]]
                e, name = members[local[m]]
                group_id[b, q] = gid
                for k, o in enumerate(e.questions[name].options):
                    canon[b, q, k] = keys.index(mapping[o])
        if gid:
            # group ids are unique within the batch; a microbatch split keeps a group whole only when its members share a window
            out["group_id"], out["canon"] = group_id, canon
        return out

    # ------------------------------------------------------------------ the loss
    def _logits(self, batch) -> Tuple[torch.Tensor, DecisionInputs]:
        inputs = DecisionInputs.from_batch(batch)
        return self.model(inputs), inputs

    def loss(self, variables, batch, step: Step):
        logits, inputs = self._logits(batch)
        B, Q, K = logits.shape
        opts = inputs.options.reshape(B * Q, K)
        lg = logits.reshape(B * Q, K)
        t = batch["targets"].reshape(B * Q, K).to(lg.device)
        scored = batch["scored"].reshape(-1).to(lg.device)
        w = batch["weights"].reshape(-1).to(lg.device)
        ordinal = inputs.ordinal.reshape(-1)
        if self.smoothing and step.train:
            k = opts.sum(-1, keepdim=True).clamp_min(1)
            t = (1 - self.smoothing) * t + self.smoothing * opts / k
        lg_safe = torch.where(opts, lg, torch.zeros_like(lg))
        charge = self.rule.charge(lg_safe, t, opts, ordinal)
        charge = torch.where(scored, charge, torch.zeros_like(charge))
        total = (charge * w).sum()
        mass = (w * scored).sum()
        p = probabilities(lg_safe, opts)
        right = ((p.argmax(-1) == t.argmax(-1)) & scored).float().sum()
        count = scored.float().sum()
        metrics = {"accuracy": Ratio(right, count.clamp_min(1))}
        if self.consistency > 0 and "group_id" in batch:
            js, n = self._consistency(p, batch["group_id"].reshape(-1).to(lg.device), batch["canon"].reshape(B * Q, K).to(lg.device), opts)
            total = total + self.consistency * js
            metrics["consistency"] = Ratio(js.detach(), n.clamp_min(1))
        return Ratio(total, mass.clamp_min(1e-12)), Aux(metrics=metrics)

    @staticmethod
    def _consistency(p, group_id, canon, opts):
        """Sum over groups and members of KL(member || mean of the members), each member's distribution on the canonical keys."""
        R, K = p.shape
        on_canon = torch.zeros(R, K, dtype=p.dtype, device=p.device).scatter_add(1, canon, p * opts)
        member = group_id > 0
        G = int(group_id.max()) + 1
        sums = torch.zeros(G, K, dtype=p.dtype, device=p.device).index_add(0, group_id, on_canon * member[:, None])
        sizes = torch.zeros(G, dtype=p.dtype, device=p.device).index_add(0, group_id, member.to(p.dtype))
        mean = (sums / sizes.clamp_min(1)[:, None])[group_id]
        kl = (on_canon * (on_canon.clamp_min(1e-12).log() - mean.clamp_min(1e-12).log())).sum(-1)
        return (kl * member).sum(), member.to(p.dtype).sum()

    # ------------------------------------------------------------------ held-out passes
    @torch.no_grad()
    def decisions(self, batch) -> Decisions:
        logits, inputs = self._logits(batch)
        B, Q, K = logits.shape
        asked = (inputs.kinds >= 0).reshape(-1)
        opts = inputs.options.reshape(B * Q, K)
        p = probabilities(torch.where(opts, logits.reshape(B * Q, K), torch.zeros_like(opts, dtype=logits.dtype)), opts)
        pick = lambda x: x.reshape(B * Q, *x.shape[2:])[asked.to(x.device)].cpu()
        return Decisions(p[asked].cpu(), pick(batch["targets"]), opts[asked].cpu(), pick(batch["scored"]),
                         inputs.ordinal.reshape(-1)[asked].cpu(), pick(batch["classes"]))

    def row_tokens(self, batch) -> Optional[int]:
        return int((batch["segment_ids"] > 0).sum())
