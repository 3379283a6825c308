"""``LMObjective``: next-token cross-entropy with a chunked head that never holds ``[tokens, vocab]`` logits for the
whole batch, packed-document masking, z-loss, optional multi-token-prediction weight, and ``Perplexity``.

Parity: src/dew/objectives/lm/objective.py:1348-1560 (arguments ``ema_decay, pad_id, head_chunks, head_tile, z_loss,
token_accuracy, loss_role ...``), src/dew/objectives/lm/chunked.py:774-874 (chunked cross-entropy).
On a GPU the head is ``ops.linear_cross_entropy``: tcgen05 GEMM tiles + a fused loss/gradient row kernel.
"""
from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from .. import ops
from .base import Aux, Exponentiated, Objective, Ratio, Step


class LMObjective(Objective):
    def __init__(self, model, seq_len: Optional[int] = None, *, ema_decay: Optional[float] = None,
                 pad_id: Optional[int] = None, head_chunks: int = 4, head_tile: Optional[int] = None,
                 z_loss: float = 0.0, token_accuracy: bool = True, variables=None, balance: Optional[float] = None,
                 mtp_weight: Optional[float] = None, prefix: Optional[int] = None, tokenizer=None, samples: Optional[dict] = None,
                 loss_role: Optional[int] = None, exit_entropy: Optional[float] = None, pass_weights=None, indexer=None, adaptation=None):
        """``samples``: preview settings ``{"prompt": [...token ids or text], "max_new_tokens": n, "sampling": Sampling}``;
        ``loss_role``: score only the targets whose ``batch["roles"]`` entry equals this role id (chat fine-tuning on the
        assistant's tokens).

        ``exit_entropy`` (beta) trains a looped decoder's exit gate: each token's loss is its cross entropy at every pass weighted
        by the probability it exits there (from the gate's hazards, the last pass taking the rest) less beta times that
        distribution's entropy; every pass's exit state is scored through the head.  ``pass_weights`` trains every pass count at
        once: ``"mean"`` or one weight per pass summing to one, each pass's term its own cross entropy (no gate needed).  The two
        are refused together.  Reports: ``ce`` (the last pass's), ``exit_ce``, ``exit_entropy`` / ``pass_<k>_ce``.

        ``indexer`` (training a sparse-attention indexer beside dense attention inside the decoder) and ``adaptation`` (in-context
        level stepping) name reference features whose model-side parts are not in this library: asking for them raises."""
        unsupported = {"indexer": indexer, "adaptation": adaptation}
        asked = [k for k, v in unsupported.items() if v is not None]
        if asked:
            raise NotImplementedError(f"LMObjective({', '.join(asked)}=...) needs an attention indexer inside the decoder / an in-context "
                                      "decoder, which this library does not provide")
        loop = getattr(getattr(model, "config", None), "loop", None)
        if exit_entropy is not None:
            if pass_weights is not None:
                raise ValueError("the exit objective weighs the passes its own way: give exit_entropy or pass_weights, not both")
            if loop is None or not loop.exit_gate or not 0 <= exit_entropy < float("inf"):
                raise ValueError("exit_entropy weighs the entropy of a looped decoder's exit distribution: it needs a model with "
                                 f"Loop(exit_gate=True) and a finite non-negative weight, got {exit_entropy}")
        if pass_weights is not None:
            if loop is None:
                raise ValueError("pass_weights train the passes of a looped decoder: the model has no loop")
            if pass_weights != "mean":
                pass_weights = tuple(float(w) for w in pass_weights)
                if len(pass_weights) != loop.steps or any(w < 0 for w in pass_weights) or abs(sum(pass_weights) - 1) > 1e-6:
                    raise ValueError(f"pass_weights are 'mean' or {loop.steps} non-negative weights summing to one")
        self.exit_entropy, self.pass_weights = exit_entropy, pass_weights
        self.samples, self.loss_role = samples, loss_role
        self.model = model
        self.seq_len = seq_len
        self.ema_decay = ema_decay
        self.pad_id = pad_id
        self.head_chunks, self.head_tile = head_chunks, head_tile
        self.z_loss = z_loss
        self.token_accuracy = token_accuracy
        self.balance = balance
        if balance is not None and not isinstance(balance, (int, float)):
            balance.prepare(model)          # an ExpertBalance: the sparse layers keep what its terms read
        self.mtp_weight = mtp_weight
        self.prefix = prefix
        self.tokenizer = tokenizer
        self._given = variables

    def init(self, key=0, variables=None):
        return super().init(key, variables if variables is not None else self._given)

    def _targets(self, batch):
        tokens = batch["tokens"]
        inputs, targets = tokens[:, :-1], tokens[:, 1:].clone()
        seg = batch.get("segments")
        seg_in = None
        if seg is not None:
            seg_in = seg[:, :-1]
            targets[(seg[:, 1:] == 0) | (seg[:, 1:] != seg[:, :-1])] = -100     # padding and document boundaries
        if self.pad_id is not None:
            targets[targets == self.pad_id] = -100
        mask = batch.get("loss_mask")
        if mask is not None:
            targets[mask[:, 1:] == 0] = -100
        if self.prefix:
            targets[:, : self.prefix] = -100
        if self.loss_role is not None and "roles" in batch:
            targets[batch["roles"][:, 1:] != self.loss_role] = -100
        return inputs, targets, seg_in

    def _pass_losses(self, variables, batch, step: Step):
        """The looped decoder's objectives: every pass's exit state scored through the head, per token."""
        import torch.nn.functional as F
        inputs, targets, seg = self._targets(batch)
        states = self.apply(variables, inputs, train=step.train, segment_ids=seg, return_hidden=True, passes=True)
        if variables is None:
            w = self.model.head_weight()
        else:
            from ..utils.trees import variables_for_call
            named = variables_for_call(self.model, variables)
            w = named[getattr(self.model, "head_parameter", None) or ("embed.weight" if self.model.head is None else "head.weight")]
        cap = getattr(self.model.config, "logit_softcap", 0.0)
        scored = (targets != -100)
        mass = scored.sum().to(torch.float32)
        ces = []
        for st in states:
            logits = ops.linear(st, w).float()
            if cap > 0:
                logits = cap * torch.tanh(logits / cap)
            ces.append(F.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), ignore_index=-100, reduction="none").reshape(targets.shape))
        ce = torch.stack(ces)                                            # [passes, B, S]
        metrics = {"ce": Ratio((ce[-1].detach() * scored).sum(), mass), "perplexity": Exponentiated(Ratio((ce[-1].detach() * scored).sum(), mass)),
                   "tokens": Ratio(mass, torch.ones((), device=mass.device))}
        if self.exit_entropy is not None:
            p = self.model.exit_distribution(states)                    # [passes, B, S]
            expected = (p * ce).sum(0)
            entropy = -(p * torch.log(p.clamp_min(1e-12))).sum(0)
            total = ((expected - self.exit_entropy * entropy) * scored).sum()
            depth = (p * torch.arange(1, len(states) + 1, device=p.device, dtype=p.dtype)[:, None, None]).sum(0)
            metrics.update(exit_ce=Ratio((expected.detach() * scored).sum(), mass), exit_entropy=Ratio((entropy.detach() * scored).sum(), mass),
                           exit_depth=Ratio((depth.detach() * scored).sum(), mass))
        else:
            k = len(states)
            weights = [1.0 / k] * k if self.pass_weights == "mean" else list(self.pass_weights)
            total = sum(wk * (ce[i] * scored).sum() for i, wk in enumerate(weights) if wk > 0)
            metrics.update({f"pass_{i + 1}_ce": Ratio((ce[i].detach() * scored).sum(), mass) for i in range(k)})
        if self.z_loss:
            logits = ops.linear(states[-1], w).float()
            total = total + self.z_loss * ((torch.logsumexp(logits, -1) ** 2) * scored).sum()
        return Ratio(total, mass), Aux(metrics=metrics)

    def loss(self, variables, batch: Mapping[str, torch.Tensor], step: Step):
        if self.exit_entropy is not None or self.pass_weights is not None:
            return self._pass_losses(variables, batch, step)
        inputs, targets, seg = self._targets(batch)
        hidden = self.apply(variables, inputs, train=step.train, segment_ids=seg, return_hidden=True)
        B, S, d = hidden.shape
        if variables is None:
            w = self.model.head_weight()
        else:
            from ..utils.trees import variables_for_call
            named = variables_for_call(self.model, variables)
            w = named[getattr(self.model, "head_parameter", None) or ("embed.weight" if self.model.head is None else "head.weight")]
        tile = self.head_tile or max(1, (B * S + self.head_chunks - 1) // self.head_chunks)
        cap = getattr(self.model.config, "logit_softcap", 0.0)
        divisor = getattr(self.model.config, "logit_divisor", 1.0)
        if divisor != 1.0:
            hidden = hidden / divisor                                       # logits = h W^T / divisor
        tp_head = getattr(self.model, "tp_head", None)
        if tp_head is not None and getattr(self.model, "tp_training", False):
            # vocabulary-parallel head: every tensor rank scores its slice of the vocabulary; maxima, sums and the target
            # logit meet in all-reduces, and the hidden state's gradient is summed over the ranks in the backward
            from ..parallel.sp_ops import vocab_parallel_cross_entropy
            from ..parallel.tp import copy_to_region
            group = self.model.tp.group
            total, mass = vocab_parallel_cross_entropy(copy_to_region(hidden.reshape(B * S, d), group), tp_head,
                                                       targets.reshape(-1), group=group, ignore_index=-100)
        else:
            total, mass = ops.linear_cross_entropy(hidden.reshape(B * S, d), w, targets.reshape(-1), ignore_index=-100,
                                                   z_loss=self.z_loss, softcap=cap, chunk=tile)
        massf = mass.to(torch.float32)
        mtp_metrics = {}
        if self.mtp_weight and getattr(self.model, "mtp", None) is not None and variables is None:
            # depth k scores token t+k+1 from position t: the main targets shifted by k, averaged over the depths
            tokens = batch["tokens"]
            depths = self.model.mtp_hiddens(hidden, tokens[:, : S + 1], seg)
            extra = hidden.new_zeros((), dtype=torch.float32)
            for k, hk in enumerate(depths, start=1):
                tk = targets[:, k:]
                lk, mk = ops.linear_cross_entropy(hk.reshape(-1, d), w, tk.reshape(-1), ignore_index=-100, softcap=cap, chunk=tile)
                mkf = mk.to(torch.float32).clamp_min(1.0)
                extra = extra + lk / mkf
                mtp_metrics[f"mtp_loss_{k}"] = Ratio(lk.detach(), mkf)
            if depths:
                total = total + self.mtp_weight * (extra / len(depths)) * massf
        aux = Aux(metrics={"perplexity": Exponentiated(Ratio(total.detach(), massf)),
                           "tokens": Ratio(massf, torch.ones((), device=massf.device)), **mtp_metrics})
        from .routing import ExpertBalance
        if isinstance(self.balance, ExpertBalance):
            # the run's router policy reads the sparse layers' records (and clears them, so pop_aux below adds nothing twice)
            routed, raux = self.balance.compose(self.model, Ratio(total, massf), batch.get("segments"))
            total = routed.total
            aux.metrics.update(raux.metrics)
            aux.effects.update(raux.effects)
        moe_aux = getattr(self.model, "pop_aux", None)
        if moe_aux is not None and not isinstance(self.balance, ExpertBalance):
            extra = moe_aux()
            aux.metrics.update(extra.get("metrics", {}))
            aux.effects.update(extra.get("effects", {}))
            if self.balance and "balance_loss" in extra:
                total = total + self.balance * extra["balance_loss"] * massf
        return Ratio(total, massf), aux

    def uniform_mass(self, batch) -> bool:
        """Whether every target of ``batch`` is scored, so that its mass follows from its shape alone (the same on every
        rank that holds a batch of this shape)."""
        return ("segments" not in batch and "loss_mask" not in batch and self.pad_id is None and not self.prefix
                and not (self.loss_role is not None and "roles" in batch))

    def scored_tokens(self, batch):
        t = batch["tokens"]
        if self.uniform_mass(batch):
            return int(t.shape[0] * (t.shape[1] - 1))        # every target is scored: no device read needed
        return int((self._targets(batch)[1] != -100).sum())

    def row_tokens(self, batch):
        t = batch["tokens"]
        return int(t.shape[0] * (t.shape[1] - 1))

    def model_flops(self, batch):
        t = batch["tokens"]
        return self.model.model_flops(t.shape[0] * (t.shape[1] - 1), t.shape[1] - 1)

    def predict(self, variables, batch):
        return self.apply(variables, batch["tokens"])

    def preview(self, variables, batch=None, key=0, **kw):
        """Text samples from the current weights (``samples`` settings): a ``TextSamples`` artifact, or None."""
        if not self.samples or not self.samples.get("max_new_tokens"):
            return None
        from ..sampling.text import Sampling, generate
        from ..utils.artifacts import TextSamples
        prompt = self.samples.get("prompt", [[0]])
        prompts = prompt if (prompt and isinstance(prompt[0], (list, tuple, str))) else [prompt]
        gen = generate(self.model, variables, prompts, int(self.samples["max_new_tokens"]), key=key,
                       sampling=self.samples.get("sampling", Sampling(temperature=0.0)), tokenizer=self.tokenizer)
        texts = gen.text if gen.text is not None else [" ".join(map(str, gen.new_tokens(r).tolist())) for r in range(len(prompts))]
        shown = [p if isinstance(p, str) else " ".join(map(str, p)) for p in prompts]
        return TextSamples(shown, texts)

    def pipeline(self, state, ema: Optional[bool] = None):
        from ..inference.tasks import TextGeneration
        variables = state.averaged if (ema or (ema is None and state.ema is not None)) else state.variables
        return TextGeneration(self.model, variables, tokenizer=self.tokenizer)


class Perplexity:
    """Metric: ``exp(mean token negative log-likelihood)`` pooled exactly over batches."""
    name = "perplexity"

    def __call__(self, objective: LMObjective, variables, batch, step: Step):
        stats, _ = objective.loss(variables, batch, step)
        return Exponentiated(stats)
