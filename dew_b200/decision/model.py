from __future__ import annotations

from typing import Dict, List, Mapping, Sequence, Tuple

import torch
import torch.nn as nn

from .questions import Question


def layout_row(state: Sequence[int], questions: Sequence[Question], marker_id: int, max_len: int, pad_id: int = 0):
    """State first, then one marker token per question (a causal backbone has read the whole state at every marker).
    Returns ``(tokens [max_len], marker positions [Q])``; the state is truncated on the left if the row is too short."""
    room = max_len - len(questions)
    state = list(state)[-room:]
    row = state + [marker_id] * len(questions)
    pos = [len(state) + i for i in range(len(questions))]
    return torch.tensor(row + [pad_id] * (max_len - len(row)), dtype=torch.long), torch.tensor(pos, dtype=torch.long)


class DecisionHead(nn.Module):
    """Scores option ``o`` of question ``q`` as ``<W_q h, e_{q,o}> + b_{q,o}``: a per-question projection of the hidden state
    at the question's marker against a learned embedding per option."""

    def __init__(self, features: int, questions: Sequence[Question], width: int = 64):
        super().__init__()
        self.questions = list(questions)
        self.proj = nn.ModuleList([nn.Linear(features, width) for _ in self.questions])
        self.options = nn.ParameterList([nn.Parameter(torch.randn(len(q.options), width) * width ** -0.5) for q in self.questions])
        self.bias = nn.ParameterList([nn.Parameter(torch.zeros(len(q.options))) for q in self.questions])

    def forward(self, hidden_at_markers: torch.Tensor) -> List[torch.Tensor]:
        """``hidden_at_markers [B, Q, d]`` -> per question, logits ``[B, options]``."""
        return [self.proj[i](hidden_at_markers[:, i].float()) @ self.options[i].t() + self.bias[i] for i in range(len(self.questions))]


class Decide(nn.Module):
    """The task: backbone + head; ``answer(states)`` returns per request a dict question name -> {option: probability}."""

    def __init__(self, backbone, questions: Sequence[Question], marker_id: int, max_len: int = 128, width: int = 64):
        super().__init__()
        self.backbone, self.questions, self.marker_id, self.max_len = backbone, list(questions), marker_id, max_len
        features = backbone.config.emb_features
        self.head = DecisionHead(features, questions, width)

    def encode(self, states: Sequence[Sequence[int]]):
        rows, pos = zip(*(layout_row(s, self.questions, self.marker_id, self.max_len) for s in states))
        return torch.stack(rows), torch.stack(pos)

    def logits(self, tokens: torch.Tensor, positions: torch.Tensor) -> List[torch.Tensor]:
        h = self.backbone.hidden(tokens)
        at = h.gather(1, positions.to(h.device)[..., None].expand(-1, -1, h.shape[-1]))
        return self.head(at)

    @torch.no_grad()
    def answer(self, states: Sequence[Sequence[int]], temperatures=None) -> List[Dict[str, Dict[str, float]]]:
        dev = next(self.parameters()).device
        tokens, pos = self.encode(states)
        logits = self.logits(tokens.to(dev), pos.to(dev))
        out = [dict() for _ in states]
        for qi, (q, lg) in enumerate(zip(self.questions, logits)):
            t = 1.0 if temperatures is None else float(temperatures.value[qi])
            probs = torch.softmax(lg / t, -1).cpu()
            for r in range(len(states)):
                out[r][q.name] = {o: float(p) for o, p in zip(q.options, probs[r])}
        return out
