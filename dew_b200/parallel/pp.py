"""Pipeline parallelism (GPipe): the layer stack is cut into ``stage`` consecutive groups, microbatches flow forward
through the stages and gradients flow back, activations moving between neighbouring ranks with point-to-point sends and
receives (NCCL p2p on GPUs).

Parity: src/dew/nn/backbones/decoder_stack.py:1468-1593 (``run_pipeline``: GPipe only - "Dew does not implement a 1F1B
schedule", docs/concepts/distributed.md:256 - microbatch_count, stage-local optimizer state), src/dew/training/stages.py.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn


def stage_slices(num_layers: int, stages: int) -> List[range]:
    """Consecutive, near-equal groups of layers (earlier stages take the remainder)."""
    base, extra = divmod(num_layers, stages)
    out, lo = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        out.append(range(lo, lo + n))
        lo += n
    return out


class GPipe:
    """Runs ``stage_fn(x) -> y`` of this rank over ``microbatches`` inputs: all forwards, then all backwards."""

    def __init__(self, stage_fn: Callable[[torch.Tensor], torch.Tensor], group: Optional[dist.ProcessGroup] = None,
                 first_input: bool = True):
        self.fn, self.group = stage_fn, group
        self.stages = dist.get_world_size(group) if dist.is_initialized() else 1
        self.stage = dist.get_rank(group) if dist.is_initialized() else 0
        self.prev = dist.get_global_rank(group, self.stage - 1) if (group is not None and self.stage > 0) else self.stage - 1
        self.next = dist.get_global_rank(group, self.stage + 1) if (group is not None and self.stage < self.stages - 1) else self.stage + 1

    def run(self, inputs: Optional[Sequence[torch.Tensor]], loss_fn: Optional[Callable[[torch.Tensor, int], torch.Tensor]],
            microbatches: int, activation_like: torch.Tensor) -> Optional[torch.Tensor]:
        """``inputs`` are given on the first stage; ``loss_fn(y, i)`` on the last. ``activation_like`` fixes the shape /
        dtype of what crosses stage boundaries. Returns the summed loss on the last stage."""
        first, last = self.stage == 0, self.stage == self.stages - 1
        acts_in: List[torch.Tensor] = []
        acts_out: List[torch.Tensor] = []
        total = None
        for i in range(microbatches):                      # forward wave
            if first:
                x = inputs[i]
            else:
                x = torch.empty_like(activation_like)
                dist.recv(x, src=self.prev, group=self.group)
                x.requires_grad_()
            y = self.fn(x)
            acts_in.append(x)
            if last:
                l = loss_fn(y, i)
                total = l if total is None else total + l
                acts_out.append(l)
            else:
                dist.send(y.detach().contiguous(), dst=self.next, group=self.group)
                acts_out.append(y)
        for i in reversed(range(microbatches)):            # backward wave
            if last:
                acts_out[i].backward()
            else:
                g = torch.empty_like(acts_out[i])
                dist.recv(g, src=self.next, group=self.group)
                acts_out[i].backward(g)
            if not first:
                dist.send(acts_in[i].grad.contiguous(), dst=self.prev, group=self.group)
        return total.detach() if total is not None else None
