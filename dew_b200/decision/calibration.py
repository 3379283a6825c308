from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch


@dataclass
class Temperatures:
    """One temperature per question, fitted on held-out logits by minimising the log score (LBFGS on log T)."""
    value: torch.Tensor

    @classmethod
    def fit(cls, logits: Sequence[torch.Tensor], answers: torch.Tensor, steps: int = 50) -> "Temperatures":
        out = []
        for qi, lg in enumerate(logits):
            y = answers[:, qi]
            live = y >= 0
            if not bool(live.any()):
                out.append(torch.tensor(1.0))
                continue
            lt = torch.zeros((), requires_grad=True)
            opt = torch.optim.LBFGS([lt], lr=0.5, max_iter=steps)
            lgd, yd = lg[live].detach().float(), y[live]
            def closure():
                opt.zero_grad()
                loss = torch.nn.functional.cross_entropy(lgd / lt.exp(), yd)
                loss.backward()
                return loss
            opt.step(closure)
            out.append(lt.detach().exp())
        return cls(torch.stack(out))


def binning(confidence: torch.Tensor, correct: torch.Tensor, bins: int = 10):
    """Reliability table: per confidence bin (count, mean confidence, accuracy) and the expected calibration error."""
    edges = torch.linspace(0, 1, bins + 1)
    rows, ece, n = [], 0.0, max(len(confidence), 1)
    for lo, hi in zip(edges[:-1], edges[1:]):
        m = (confidence > lo) & (confidence <= hi)
        c = int(m.sum())
        if c:
            conf, acc = float(confidence[m].mean()), float(correct[m].float().mean())
            ece += c / n * abs(conf - acc)
            rows.append((c, conf, acc))
        else:
            rows.append((0, 0.0, 0.0))
    return rows, ece


@dataclass
class Abstention:
    """Answer only when the top probability reaches ``threshold``; ``coverage_accuracy`` reports the trade-off."""
    threshold: float = 0.5

    def decide(self, probs: torch.Tensor):
        top, idx = probs.max(-1)
        return torch.where(top >= self.threshold, idx, torch.full_like(idx, -1))

    def coverage_accuracy(self, probs: torch.Tensor, answers: torch.Tensor):
        d = self.decide(probs)
        kept = d >= 0
        cov = float(kept.float().mean())
        acc = float((d[kept] == answers[kept]).float().mean()) if bool(kept.any()) else 0.0
        return cov, acc
