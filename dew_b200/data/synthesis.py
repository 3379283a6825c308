"""Training data made from a model's own samples: best-of-n selection for supervised fine-tuning and chosen / rejected pairs for
preference optimisation, with what made each record written beside it.

``scored_samples(generate, prompts, n, reward)``  n completions per prompt with their rewards
``best_of_n(samples, minimum)``                    per prompt the highest-reward completion (ties: the shortest), dropped below ``minimum``
``preference_pairs(samples, margin, per_prompt)``  (chosen, rejected) from each prompt's completions whose rewards differ by at least
                                                   ``margin``; identical completions never pair; the largest gaps first
``sft_rows`` / ``dpo_rows``                        token rows with loss masks in the shape the ``sft`` and ``preferences`` presets read
``write_records``                                  JSON lines with provenance (the generator's name, the sampling settings, the reward's name)

Reference: the rejection-sampling and preference-data steps of recipes/chain.py and src/dew/data/preferences.py (pair records with
``chosen_mask`` / ``rejected_mask``).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import numpy as np


@dataclass
class Sample:
    prompt: Tuple[int, ...]
    completion: Tuple[int, ...]
    reward: float
    index: int = 0                     # the prompt's index in its source
    draw: int = 0                      # which of the n draws


def scored_samples(generate: Callable[[Sequence[Sequence[int]], int], Sequence[Sequence[Sequence[int]]]], prompts: Sequence[Sequence[int]], n: int,
                   reward: Callable[[Sequence[int], Sequence[int]], float]) -> List[Sample]:
    """``generate(prompts, n)`` returns, per prompt, ``n`` completions (token ids)."""
    out = []
    for i, (p, completions) in enumerate(zip(prompts, generate(prompts, n))):
        if len(completions) != n:
            raise ValueError(f"prompt {i}: asked for {n} completions, got {len(completions)}")
        for d, c in enumerate(completions):
            out.append(Sample(tuple(p), tuple(c), float(reward(p, c)), i, d))
    return out


def _by_prompt(samples: Iterable[Sample]) -> Dict[int, List[Sample]]:
    groups: Dict[int, List[Sample]] = {}
    for s in samples:
        groups.setdefault(s.index, []).append(s)
    return groups


def best_of_n(samples: Iterable[Sample], minimum: Optional[float] = None) -> List[Sample]:
    out = []
    for i, group in sorted(_by_prompt(samples).items()):
        best = min(group, key=lambda s: (-s.reward, len(s.completion), s.draw))
        if minimum is None or best.reward >= minimum:
            out.append(best)
    return out


def preference_pairs(samples: Iterable[Sample], margin: float = 0.0, per_prompt: int = 1) -> List[Tuple[Sample, Sample]]:
    out = []
    for i, group in sorted(_by_prompt(samples).items()):
        pairs = [(a, b) for a in group for b in group if a.reward - b.reward > margin and a.completion != b.completion]
        pairs.sort(key=lambda ab: (-(ab[0].reward - ab[1].reward), ab[0].draw, ab[1].draw))
        used_a, used_b, taken = set(), set(), 0
        for a, b in pairs:
            if taken >= per_prompt:
                break
            if a.draw in used_a or b.draw in used_b:                          # each completion chosen once and rejected once at most
                continue
            out.append((a, b))
            used_a.add(a.draw); used_b.add(b.draw)
            taken += 1
    return out


def _row(prompt: Sequence[int], completion: Sequence[int], length: int, pad_id: int) -> Tuple[np.ndarray, np.ndarray]:
    ids = (list(prompt) + list(completion))[:length]
    tokens = np.full(length, pad_id, dtype=np.int64)
    tokens[: len(ids)] = ids
    mask = np.zeros(length, dtype=np.float32)
    mask[min(len(prompt), length): len(ids)] = 1.0
    return tokens, mask


def sft_rows(samples: Iterable[Sample], seq_len: int, pad_id: int = 0) -> Dict[str, np.ndarray]:
    rows = [_row(s.prompt, s.completion, seq_len + 1, pad_id) for s in samples]
    return {"tokens": np.stack([t for t, _ in rows]), "loss_mask": np.stack([m for _, m in rows])}


def dpo_rows(pairs: Iterable[Tuple[Sample, Sample]], seq_len: int, pad_id: int = 0) -> Dict[str, np.ndarray]:
    pairs = list(pairs)
    c = [_row(a.prompt, a.completion, seq_len + 1, pad_id) for a, _ in pairs]
    r = [_row(b.prompt, b.completion, seq_len + 1, pad_id) for _, b in pairs]
    return {"chosen": np.stack([t for t, _ in c]), "chosen_mask": np.stack([m for _, m in c]),
            "rejected": np.stack([t for t, _ in r]), "rejected_mask": np.stack([m for _, m in r])}


def write_records(path: str, records: Iterable[Any], provenance: Optional[Mapping[str, Any]] = None) -> int:
    """Samples or (chosen, rejected) pairs as JSON lines; the first line of the file is the provenance record."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    n = 0
    with open(path + ".tmp", "w") as f:
        f.write(json.dumps({"provenance": dict(provenance or {})}) + "\n")
        for rec in records:
            if isinstance(rec, tuple):
                a, b = rec
                row = {"prompt": list(a.prompt), "chosen": list(a.completion), "rejected": list(b.completion), "chosen_reward": a.reward,
                       "rejected_reward": b.reward, "index": a.index}
            else:
                row = {"prompt": list(rec.prompt), "completion": list(rec.completion), "reward": rec.reward, "index": rec.index, "draw": rec.draw}
            f.write(json.dumps(row) + "\n")
            n += 1
    os.replace(path + ".tmp", path)
    return n
