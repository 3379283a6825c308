"""The mean of runs' weights.  ``mean_of`` averages variable trees leaf by leaf (fp32 accumulation, each leaf back in its own dtype;
integer leaves - step counters, token tables - are the first tree's); ``average_steps`` averages the last few steps of one run
(the tail average that stands in for a learning-rate cooldown); ``greedy_soup`` adds candidates, best first, for as long as the mean
scores no worse (Wortsman et al., "Model soups", arXiv 2203.05482).  Trees whose paths or shapes differ raise naming the path: averaging
models of different architectures is never what was meant.

Reference: src/dew/checkpoints/averaging.py.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..utils.trees import flatten, unflatten


def mean_of(trees: Sequence[Mapping[str, Any]], weights: Optional[Sequence[float]] = None) -> Dict[str, Any]:
    if not trees:
        raise ValueError("the mean of no trees")
    w = [1.0 / len(trees)] * len(trees) if weights is None else [float(x) / float(sum(weights)) for x in weights]
    if len(w) != len(trees):
        raise ValueError(f"{len(trees)} trees and {len(w)} weights")
    flats = [flatten(t) for t in trees]
    first = flats[0]
    out: Dict[str, Any] = {}
    for path, leaf in first.items():
        for i, f in enumerate(flats[1:], 1):
            if path not in f:
                raise KeyError(f"tree {i} holds no {path!r}")
            if torch.is_tensor(leaf) and tuple(f[path].shape) != tuple(leaf.shape):
                raise ValueError(f"{path!r} is {tuple(leaf.shape)} in tree 0 and {tuple(f[path].shape)} in tree {i}")
        if torch.is_tensor(leaf) and leaf.is_floating_point():
            acc = torch.zeros_like(leaf, dtype=torch.float32)
            for wi, f in zip(w, flats):
                acc.add_(f[path].detach().to(acc.device, torch.float32), alpha=wi)
            out[path] = acc.to(leaf.dtype)
        else:
            out[path] = leaf
    for i, f in enumerate(flats[1:], 1):
        extra = sorted(set(f) - set(first))
        if extra:
            raise KeyError(f"tree {i} holds {extra[:3]} that tree 0 does not")
    return unflatten(out)


def average_steps(checkpoints, steps: Optional[Sequence[int]] = None, last: Optional[int] = None, ema: Optional[bool] = None) -> Dict[str, Any]:
    """The mean of a run's variables over ``steps``, or over its ``last`` saved steps."""
    if steps is None:
        saved = checkpoints.steps()
        if not saved:
            raise FileNotFoundError("the run has saved no steps")
        steps = saved[-(last or len(saved)):]
    return mean_of([checkpoints.variables(step=s, ema=ema) for s in steps])


def greedy_soup(candidates: Sequence[Mapping[str, Any]], score: Callable[[Mapping[str, Any]], float], higher_is_better: bool = True
                ) -> Tuple[Dict[str, Any], List[int], float]:
    """``(soup, indices of the candidates in it, its score)``: candidates are ranked by their own score; each joins the soup if the mean
    with it scores at least as well as the soup without it."""
    sign = 1.0 if higher_is_better else -1.0
    own = [sign * float(score(c)) for c in candidates]
    order = sorted(range(len(candidates)), key=lambda i: -own[i])
    chosen = [order[0]]
    soup, best = mean_of([candidates[order[0]]]), own[order[0]]
    for i in order[1:]:
        trial = mean_of([candidates[j] for j in chosen + [i]])
        s = sign * float(score(trial))
        if s >= best:
            chosen, soup, best = chosen + [i], trial, s
    return soup, chosen, sign * best
