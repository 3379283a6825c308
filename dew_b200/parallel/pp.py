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


class PipelineEngine:
    """Training engine for a mesh with ``stage > 1``: consecutive layers of a ``CausalTransformer`` live on consecutive
    stage ranks, microbatches flow forward and gradients back (GPipe), and every stage keeps the fp32 parameters and the
    optimizer state of its own layers only (stage-local state: src/dew/training/stages.py; schedule:
    src/dew/nn/backbones/decoder_stack.py:1499-1593).

    Transfers are NCCL (or gloo) point-to-point operations issued in groups - the send of microbatch ``i``'s output together
    with the receive of microbatch ``i + 1``'s input - so they run on the backend's own streams while this stage computes;
    the compute stream waits only for the receive it is about to consume.  With a ``data`` axis beside ``stage`` the
    gradients of each stage are summed over its data-parallel peers before the update."""

    def __init__(self, trainer, mesh):
        self.t, self.mesh = trainer, mesh
        self.model = trainer.objective.model
        self.group = mesh.group("stage")
        self.stages = mesh.sizes["stage"]
        self.stage = mesh.index("stage")
        batch_axes = tuple(a for a in ("data", "expert", "fsdp") if mesh.sizes[a] > 1)
        self.batch_group = mesh.group(*batch_axes) if batch_axes else None
        self.batch_ranks = mesh.size(*batch_axes) if batch_axes else 1
        self.batch_index = mesh.index(*batch_axes) if batch_axes else 0
        ranks = mesh.axis_ranks(("stage",))
        self.prev = ranks[self.stage - 1] if self.stage > 0 else None
        self.next = ranks[self.stage + 1] if self.stage < self.stages - 1 else None
        self.first, self.last = self.stage == 0, self.stage == self.stages - 1
        layers = self.model.layers
        self.mine = stage_slices(len(layers), self.stages)[self.stage]
        self._trimmed = False

    # ------------------------------------------------------------------ state
    def _own_modules(self):
        mods = [self.model.layers[i] for i in self.mine]
        if self.first:
            mods.append(self.model.embed)
        if self.last:
            mods.append(self.model.final_norm)
            if self.model.head is not None:
                mods.append(self.model.head)
            elif not self.first:
                mods.append(self.model.embed)              # tied head: the last stage holds its own copy of the table
        return mods

    def _own_named(self):
        own = {id(p) for m in self._own_modules() for p in m.parameters()}
        return [(n, p) for n, p in self.model.named_parameters() if id(p) in own]

    def fresh_state(self, key: int):
        from ..nn.layers import reset_all
        from ..training.state import TrainState
        from ..utils import keys as K
        from ..utils.trees import module_path_to_tree_path, unflatten
        reset_all(self.model, int(K.fold_in(key, "init")) & 0x7FFFFFFF)        # every stage draws the whole model alike ...
        if not self._trimmed:
            own = {id(p) for _, p in self._own_named()}
            for mod in self.model.modules():                                      # ... and keeps its own part
                for name, p in list(mod._parameters.items()):
                    if p is not None and id(p) not in own:
                        mod._parameters[name] = nn.Parameter(torch.empty(0, dtype=p.dtype, device=p.device), requires_grad=False)
            self._trimmed = True
        params = {module_path_to_tree_path(n): p for n, p in self._own_named()}
        variables = {"params": unflatten(params)}
        state = TrainState(variables=variables, opt_state=self.t.optimizer.init(variables["params"]), key=key)
        if self.t.objective.ema_spec() is not None:
            from ..utils.trees import tree_map
            state.ema = {"params": tree_map(lambda x: x.detach().clone(), variables["params"])}
        return state

    def adopt(self, state):
        return state

    # ------------------------------------------------------------------ one stage's forward
    def _stage_forward(self, x, mb):
        m = self.model
        cfg = m.config
        if self.first:
            h = m.embed(mb["tokens"][:, :-1])
            if cfg.embed_scale:
                h = h * (cfg.emb_features ** 0.5)
        else:
            h = x
        cos, sin = m.rope_tables(h.device)
        branch = None
        for i in self.mine:
            h, branch = m.layers[i](h, branch, cos, sin, None, None, None)
        if self.last:
            n, _ = m.final_norm(h, branch)
            return n
        return h if branch is None else h + branch          # the pending branch is folded in at the stage boundary

    def _loss(self, hidden, mb):
        from .. import ops
        B, S, d = hidden.shape
        targets = mb["tokens"][:, 1:]
        total, mass = ops.linear_cross_entropy(hidden.reshape(B * S, d), self.model.head_weight(), targets.reshape(-1),
                                               ignore_index=-100, chunk=max(1, B * S // 4))
        return total, mass

    # ------------------------------------------------------------------ the step
    def step(self, state, batch):
        from ..objectives.base import Ratio
        from ..training.trainer import _split_rows
        from ..utils.trees import flatten, module_path_to_tree_path, unflatten
        t = self.t
        M = t.microbatches or self.stages
        parts = _split_rows(batch, M)
        dev = next(p for _, p in self._own_named()).device
        rows, S = parts[0]["tokens"].shape[0], parts[0]["tokens"].shape[1] - 1
        d = self.model.config.emb_features
        dtype = next(p for _, p in self._own_named()).dtype
        for _, p in self._own_named():
            p.grad = None
        acts_in, acts_out = [None] * M, [None] * M
        total_loss = torch.zeros((), dtype=torch.float32, device=dev)
        total_mass = torch.zeros((), dtype=torch.float32, device=dev)

        def post(send, send_to, recv_shape, recv_from):
            """One grouped point-to-point round: returns (received tensor or None, requests)."""
            ops_, got = [], None
            if send is not None:
                ops_.append(dist.P2POp(dist.isend, send, send_to))
            if recv_shape is not None:
                got = torch.empty(recv_shape, dtype=dtype, device=dev)
                ops_.append(dist.P2POp(dist.irecv, got, recv_from))
            return got, (dist.batch_isend_irecv(ops_) if ops_ else [])

        shape = (rows, S, d)
        # ---- forward wave
        nxt, reqs = post(None, None, None if self.first else shape, self.prev)
        keep = []                                           # sent tensors stay alive until their sends complete
        for i in range(M):
            for r in reqs:
                r.wait()
            x = nxt
            if x is not None:
                x.requires_grad_()
            y = self._stage_forward(x, parts[i])
            acts_in[i] = x
            if self.last:
                l, mass = self._loss(y, parts[i])
                acts_out[i] = l
                total_loss += l.detach()
                total_mass += mass.detach().float()
                out = None
            else:
                acts_out[i] = y
                out = y.detach().contiguous()
                keep.append(out)
            more = i + 1 < M
            nxt, reqs = post(out, self.next, shape if (more and not self.first) else None, self.prev)
            if not more:
                for r in reqs:
                    r.wait()
        # the pooled mass scales every gradient: known on the last stage, sent to all
        stats = torch.stack([total_loss, total_mass])
        dist.broadcast(stats, src=self.mesh.axis_ranks(("stage",))[-1], group=self.group)
        if self.batch_group is not None:
            dist.all_reduce(stats, group=self.batch_group)
        mass_all = float(stats[1])
        # ---- backward wave (reverse order; gradients flow to the previous stage)
        g_in, reqs = post(None, None, None if self.last else shape, self.next)
        for i in reversed(range(M)):
            for r in reqs:
                r.wait()
            if self.last:
                acts_out[i].backward()
            else:
                acts_out[i].backward(g_in)
            gx = None if self.first else acts_in[i].grad.contiguous()
            if gx is not None:
                keep.append(gx)
            more = i > 0
            g_in, reqs = post(gx, self.prev, shape if (more and not self.last) else None, self.next)
            if not more:
                for r in reqs:
                    r.wait()
            acts_out[i] = acts_in[i] = None
        # ---- stage-local update
        named = self._own_named()
        if self.batch_group is not None:
            for _, p in named:
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.batch_group)
        if self.model.head is None and self.stages > 1 and (self.first or self.last):
            # a tied embedding lives on the first and the last stage: their gradients are summed so both copies stay equal
            pair = dist.new_group([self.mesh.axis_ranks(("stage",))[0], self.mesh.axis_ranks(("stage",))[-1]]) if not hasattr(self, "_tied") else self._tied
            self._tied = pair
            g = self.model.embed.weight.grad
            dist.all_reduce(g, group=pair)
        grads = unflatten({module_path_to_tree_path(n): p.grad for n, p in named if p.grad is not None})
        new_opt, info = t.optimizer.update(state.variables["params"], grads, state.opt_state, state.step,
                                           grad_scale=1.0 / max(mass_all, 1e-12))
        skipped = bool(info.get("skipped", False))
        if state.ema is not None and not skipped:
            from ..optim import ema_update
            ema_update(state.ema["params"], state.variables["params"], t.objective.ema_spec().at(state.updates + 1))
        rows_total = rows * M * self.batch_ranks
        new_state = state.replace(step=state.step + 1, microstep=state.microstep + M, updates=state.updates + (0 if skipped else 1),
                                  opt_state=new_opt,
                                  consumed={"examples": state.consumed.get("examples", 0) + rows_total,
                                            "tokens": state.consumed.get("tokens", 0) + rows_total * S})
        loss = Ratio(stats[0].clone(), stats[1].clone())
        return new_state, {"loss": loss, **info}
