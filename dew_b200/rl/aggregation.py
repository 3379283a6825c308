"""A student's own steps labelled by a privileged teacher and aggregated into what the student learns from: DAgger (Ross, Gordon
and Bagnell, arXiv 1011.0686), for any teacher policy and any student policy over one environment.

A student cloned from a teacher's episodes alone learns the teacher's actions at the teacher's states; its own errors take it to
states those episodes never reached, where its errors grow.  Here the student acts, so its data holds the states its own errors
lead to, and at each of them the teacher - reading what the student cannot (a privileged view of the true state) - answers the
action it would take there: the step's label.  ``labelled`` writes each label beside its step (``extras[LABEL]``); ``mixed`` lets
the teacher act with probability ``beta`` (DAgger's mixture policy, annealed toward the student).

Reference: src/dew/rl/aggregation.py (``Teacher``, ``labelled``, ``paired``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Tuple

import torch

LABEL = "label"


@dataclass
class Teacher:
    policy: Callable          # a ``Policy`` over the same step, reading its own (privileged) views
    variables: Any = None


def paired(student_variables, teacher: Teacher) -> Dict[str, Any]:
    return {"student": student_variables, "teacher": teacher.variables}


def labelled(student: Callable, teacher: Teacher, beta: float = 0.0) -> Callable:
    """A policy over ``paired`` variables: the student acts from the step and its memory; the teacher's action at the same step is
    written under ``extras[LABEL]``.  With ``beta > 0`` each environment's executed action is the teacher's with probability
    ``beta`` (drawn from the step's key), the student's otherwise; ``extras['teacher_acted']`` says which."""
    def policy(variables, observation, memory, key):
        action, extras, memory = student(variables["student"], observation, memory, key)
        with torch.no_grad():
            label, _, _ = teacher.policy(variables["teacher"], observation, None, key)
        extras = {**extras, LABEL: label}
        if beta > 0:
            g = torch.Generator().manual_seed(int(key) & 0x7FFFFFFF)
            pick = (torch.rand(action.shape[0], generator=g) < beta).to(action.device)
            action = torch.where(pick.reshape(-1, *([1] * (action.dim() - 1))), label.to(action.dtype), action)
            extras["teacher_acted"] = pick
        return action, extras, memory
    return policy


def imitation_loss(predicted: torch.Tensor, label: torch.Tensor, mask: torch.Tensor = None) -> torch.Tensor:
    """Mean squared error of the student's action against the teacher's label over the kept steps."""
    err = ((predicted - label.detach()) ** 2).sum(-1)
    if mask is None:
        return err.mean()
    m = mask.to(err.dtype)
    return (err * m).sum() / m.sum().clamp_min(1)
