"""Gauss-Newton's update, damped as Levenberg-Marquardt's: a step solves

    delta = (J^T J + damping I)^-1 J^T r        (or the dual J^T (J J^T + damping I)^-1 r when there are fewer residuals)

for the residuals ``r(theta)`` and their Jacobian ``J`` in the trained parameters.  The system is formed densely in the
parameters' dtype, so it fits models whose smaller side (parameters or residuals) squared fits in memory: a physics-informed
network's, not a language model's.  ``LevenbergMarquardt.step`` accepts a step only if it lowers ``|r|^2`` and adapts the
damping (divide after an accepted step, multiply after a rejected one).

Reference: src/dew/gauss_newton.py (``NormalEquations`` / ``RowEquations``, one solve per update), examples/pinn_burgers.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Mapping, Tuple

import torch


def _flatten(tree: Mapping[str, torch.Tensor]) -> torch.Tensor:
    return torch.cat([tree[k].reshape(-1) for k in sorted(tree)])


def _unflatten(vec: torch.Tensor, like: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out, at = {}, 0
    for k in sorted(like):
        n = like[k].numel()
        out[k] = vec[at:at + n].reshape(like[k].shape)
        at += n
    return out


def jacobian(residuals: Callable[[Mapping[str, torch.Tensor]], torch.Tensor], params: Mapping[str, torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(r [m], J [m, n])`` with the parameters flattened in sorted-name order."""
    r = residuals(params)
    jac = torch.func.jacrev(residuals)(dict(params))
    J = torch.cat([jac[k].reshape(r.shape[0], -1) for k in sorted(params)], 1)
    return r.detach(), J.detach()


def gauss_newton_direction(r: torch.Tensor, J: torch.Tensor, damping: float) -> torch.Tensor:
    """The damped step ``delta`` (to be subtracted from the parameters): the primal normal equations when the residuals are
    at least the parameters, the dual otherwise."""
    m, n = J.shape
    if m >= n:
        A = J.t() @ J + damping * torch.eye(n, dtype=J.dtype, device=J.device)
        return torch.linalg.solve(A, J.t() @ r)
    A = J @ J.t() + damping * torch.eye(m, dtype=J.dtype, device=J.device)
    return J.t() @ torch.linalg.solve(A, r)


@dataclass
class LevenbergMarquardt:
    damping: float = 1e-2
    grow: float = 4.0
    shrink: float = 0.5
    min_damping: float = 1e-10
    max_damping: float = 1e8

    @torch.no_grad()
    def step(self, module: torch.nn.Module, residuals: Callable[[Mapping[str, torch.Tensor]], torch.Tensor]) -> Dict[str, float]:
        """One update of ``module``'s parameters in place.  ``residuals(params)`` evaluates the residual vector with the
        module called functionally on ``params`` (``torch.func.functional_call``)."""
        params = {k: v.detach() for k, v in module.named_parameters()}
        with torch.enable_grad():
            r, J = jacobian(residuals, params)
        before = float((r * r).sum())
        theta = _flatten(params)
        for _ in range(12):
            delta = gauss_newton_direction(r, J, self.damping)
            trial = _unflatten(theta - delta, params)
            after = float((residuals(trial) ** 2).sum())
            if after < before:
                for k, p in module.named_parameters():
                    p.copy_(trial[k])
                self.damping = max(self.damping * self.shrink, self.min_damping)
                return {"loss": after, "before": before, "damping": self.damping, "accepted": 1.0}
            self.damping = min(self.damping * self.grow, self.max_damping)
        return {"loss": before, "before": before, "damping": self.damping, "accepted": 0.0}
