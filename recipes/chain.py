"""A recipe chains pre-training, supervised fine-tuning, preference optimisation and online RL stages over one model.

A ``Recipe`` is an ordered sequence of ``Stage`` s sharing one decoder.  Each stage trains its own data with its own objective in
its own checkpoint directory (``<directory>/<index>-<name>``), and every stage after the first starts from the weights the stage
before it left - held in memory, nothing reloaded by hand.  The optimizer starts fresh in every stage; a stage never resumes
another stage's step count.  A GRPO stage names its reward callable; callables do not survive a command line, so a chain is a
Python value built where the reward lives:

    recipe = Recipe(model, [Stage("pretrain", "lm", data=batches, steps=1000),
                            Stage("sft", "sft", data=chat_batches, steps=200),
                            Stage("prefer", "dpo", data=pair_batches, steps=100, options={"beta": 0.1}),
                            Stage("rl", "grpo", prompts=prompts, reward=reward, steps=50, options={"group": 4})], "runs/chain")
    report = recipe.run()

Stage kinds: ``lm`` (next-token loss on ``tokens``), ``sft`` (the same loss under a ``loss_mask``), ``distill`` (KL to a frozen
``teacher`` mixed with the stage's own loss), ``dpo`` (``chosen`` / ``rejected`` pairs against the stage's starting weights as the
reference), ``grpo`` (sampled completions of ``prompts`` scored by ``reward(prompt_ids, completion_ids) -> float``, any update rule
of ``dew_b200.rl.surrogate``).  Counterpart of the reference's recipes/chain.py.
"""
from __future__ import annotations

import copy
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Mapping, Optional, Sequence

import torch

import dew_b200 as dew
from dew_b200.checkpoints import Checkpoints
from dew_b200.objectives.distillation import Distillation
from dew_b200.objectives.lm import LMObjective
from dew_b200.objectives.rl import DPO, GRPO
from dew_b200.sampling.text import Sampling, generate

KINDS = ("lm", "sft", "distill", "dpo", "grpo")


@dataclass
class Stage:
    name: str
    kind: str
    data: Optional[Iterable[Mapping[str, torch.Tensor]]] = None      # batches (lm / sft / distill / dpo)
    steps: int = 100
    optimizer: Optional[dew.OptimConfig] = None
    options: Dict[str, Any] = field(default_factory=dict)
    # grpo
    prompts: Optional[Sequence[Sequence[int]]] = None
    reward: Optional[Callable[[Sequence[int], Sequence[int]], float]] = None
    max_new_tokens: int = 8
    prompts_per_round: int = 8
    updates_per_round: int = 2
    teacher: Optional[torch.nn.Module] = None                        # distill

    def __post_init__(self):
        if self.kind not in KINDS:
            raise ValueError(f"a stage's kind is one of {KINDS}, got {self.kind!r}")
        if self.kind == "grpo" and (self.prompts is None or self.reward is None):
            raise ValueError("a grpo stage needs prompts and a reward callable")
        if self.kind == "distill" and self.teacher is None:
            raise ValueError("a distill stage needs a teacher")
        if self.kind != "grpo" and self.data is None:
            raise ValueError(f"a {self.kind} stage needs data")


def rollout_batch(model, prompts: Sequence[Sequence[int]], reward, group: int, max_new_tokens: int, key: int, device,
                  sampling: Optional[Sampling] = None) -> Dict[str, torch.Tensor]:
    """``group`` sampled completions per prompt, their rewards, and the sampler's own log-probabilities of the sampled tokens."""
    sampling = sampling or Sampling(temperature=1.0)
    rows = [list(p) for p in prompts for _ in range(group)]
    was = model.training
    model.eval()
    with torch.no_grad():
        out = generate(model, None, rows, max_new_tokens, sampling=sampling, key=key)
        width = int(out.lengths.max())
        tokens = out.tokens[:, :width].to(device)
        mask = torch.zeros(len(rows), width, device=device)
        rewards = torch.zeros(len(rows))
        for i, p in enumerate(rows):
            n = int(out.lengths[i])
            mask[i, len(p):n] = 1
            rewards[i] = float(reward(p, out.tokens[i, len(p):n].tolist()))
        logits = model(tokens[:, :-1])
        old = torch.log_softmax(logits.float(), -1).gather(-1, tokens[:, 1:, None]).squeeze(-1)
    model.train(was)
    return {"tokens": tokens, "mask": mask, "rewards": rewards.to(device), "old_logprobs": old}


@dataclass
class Recipe:
    model: torch.nn.Module
    stages: Sequence[Stage]
    directory: Optional[str] = None
    key: int = 0
    log_every: int = 10 ** 9

    def _objective(self, stage: Stage, seq_len: Optional[int]):
        opts = dict(stage.options)
        if stage.kind in ("lm", "sft"):
            obj = LMObjective(self.model, seq_len or opts.pop("seq_len", 0) or None, ema_decay=None, **opts)
            obj.starts_from_model = True
            return obj
        if stage.kind == "distill":
            obj = Distillation(self.model, stage.teacher, **opts)
            obj.starts_from_model = True
            return obj
        if stage.kind == "dpo":
            return DPO(self.model, **opts)
        return GRPO(self.model, **opts)

    def run(self) -> List[Dict[str, Any]]:
        report = []
        device = next(self.model.parameters()).device
        for index, stage in enumerate(self.stages):
            ckpt = None
            if self.directory:
                ckpt = Checkpoints(os.path.join(self.directory, f"{index}-{stage.name}"))
            optim = stage.optimizer or dew.OptimConfig(learning_rate=3e-4, weight_decay=0.0)
            tracker = dew.MemoryTracker()
            if stage.kind == "grpo":
                objective = self._objective(stage, None)
                trainer = dew.Trainer(objective, optim, key=self.key + index, checkpoints=ckpt, tracker=tracker)
                state, rewards = None, []
                g = torch.Generator().manual_seed(self.key + index)
                rounds = max(1, stage.steps // stage.updates_per_round)
                for r in range(rounds):
                    pick = torch.randint(0, len(stage.prompts), (stage.prompts_per_round,), generator=g).tolist()
                    batch = rollout_batch(self.model, [stage.prompts[i] for i in pick], stage.reward, objective.group, stage.max_new_tokens,
                                          key=(self.key + index) * 100003 + r, device=device)
                    rewards.append(float(batch["rewards"].mean()))
                    state = trainer.fit([batch] * stage.updates_per_round, state=state, steps=stage.updates_per_round * (r + 1), log_every=self.log_every)
                k = max(1, len(rewards) // 4)
                report.append({"stage": stage.name, "kind": stage.kind, "steps": rounds * stage.updates_per_round,
                               "reward_first": sum(rewards[:k]) / k, "reward_last": sum(rewards[-k:]) / k})
            else:
                first = next(iter(stage.data))
                seq_len = first["tokens"].shape[1] - 1 if "tokens" in first else None
                objective = self._objective(stage, seq_len)
                trainer = dew.Trainer(objective, optim, key=self.key + index, checkpoints=ckpt, tracker=tracker)
                data = stage.data

                def cycle(batches=data):
                    while True:
                        seen = False
                        for b in batches:
                            seen = True
                            yield {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in b.items()}
                        if not seen:
                            return
                trainer.fit(cycle(), steps=stage.steps, log_every=max(1, stage.steps // 4))
                rows = tracker.rows
                report.append({"stage": stage.name, "kind": stage.kind, "steps": stage.steps, "loss_first": rows[0]["loss"] if rows else None,
                               "loss_last": rows[-1]["loss"] if rows else None})
            if ckpt is not None:
                ckpt.wait() if hasattr(ckpt, "wait") else None
        return report
