"""What a fit sums between its logs: device-resident counters the step loop adds to without waiting on a number.

``Book`` holds the running sums on the device (loss, scored mass, finite steps, steps, tokens, work, the current run of
non-finite losses); ``bookkeep`` adds one step to it in place (a handful of tiny device ops, no host read); ``Interval``
owns a book per cadence (logging, checkpointing), reads one only when its cadence falls due - after the next step has
been dispatched - and restarts it; ``TokenClock`` tracks the tokens a run has consumed and the tokens its committed
updates trained on, which is what token-denominated budgets and cooldown points are measured against.

Reference: src/dew/training/interval.py (``Book`` :87, ``bookkeep`` :169, ``Streak`` :77, ``Interval`` :201, ``TokenClock`` :451,
``BAD_LOSS_STEPS``), checkpoint control fields ``committed_tokens`` / ``consumed_examples``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

BAD_LOSS_STEPS = 5                 # consecutive non-finite losses that stop a run
COMMITTED_TOKENS = "committed_tokens"
CONSUMED_EXAMPLES = "consumed_examples"


class NonFiniteLoss(RuntimeError):
    pass


@dataclass
class Streak:
    """Non-finite losses in a row (now) and in total since the book was restarted."""
    current: int
    total: int


class Book:
    """Running sums on the device.  Layout of ``sums``: [loss total, loss mass, finite steps, steps, tokens, flops,
    non-finite streak, non-finite total]."""
    FIELDS = ("loss_total", "loss_mass", "finite", "steps", "tokens", "flops", "streak", "nonfinite")

    def __init__(self, device="cpu"):
        self.sums = torch.zeros(len(self.FIELDS), dtype=torch.float64 if torch.device(device).type == "cpu" else torch.float32,
                                device=device)

    def restart(self, keep_streak: bool = True) -> None:
        streak = self.sums[6].clone()
        self.sums.zero_()
        if keep_streak:
            self.sums[6] = streak

    def read(self) -> Dict[str, float]:
        """One host read of every counter."""
        return dict(zip(self.FIELDS, self.sums.tolist()))


def bookkeep(book: Book, loss_total: torch.Tensor, loss_mass: torch.Tensor, tokens: int = 0, flops: float = 0.0) -> None:
    """Add one step: ``loss_total / loss_mass`` is the step's mean loss.  A non-finite step adds nothing to the loss sums,
    extends the streak, and is counted; a finite one ends the streak.  No host synchronisation."""
    s = book.sums
    lt = loss_total.detach().to(s.dtype).reshape(())
    lm = torch.as_tensor(loss_mass, device=s.device).detach().to(s.dtype).reshape(())
    ok = torch.isfinite(lt) & torch.isfinite(lm)
    okf = ok.to(s.dtype)
    zero = torch.zeros((), dtype=s.dtype, device=s.device)
    s[0] += torch.where(ok, lt, zero)
    s[1] += torch.where(ok, lm, zero)
    s[2] += okf
    s[3] += 1
    s[4] += tokens
    s[5] += flops
    s[6] = (s[6] + 1) * (1 - okf)
    s[7] += 1 - okf


def streak_of(book: Book) -> Streak:
    r = book.read()
    return Streak(int(r["streak"]), int(r["nonfinite"]))


def checked_finite(streak: Streak, step: int, *, skips: bool, limit: int = BAD_LOSS_STEPS) -> None:
    """Raise when the loss has been non-finite for ``limit`` steps in a row (or at once when non-finite steps are not
    skipped by the optimizer)."""
    if streak.current >= (limit if skips else 1):
        raise NonFiniteLoss(f"loss non-finite for {streak.current} consecutive step(s) at step {step}")


@dataclass
class TokenClock:
    """Tokens and examples of a run: ``consumed`` counts every dispatched batch, ``committed`` what finished optimizer updates
    trained on (they differ under gradient accumulation and skipped non-finite updates)."""
    consumed_tokens: int = 0
    consumed_examples: int = 0
    committed_tokens: int = 0
    pending_tokens: int = 0

    def dispatched(self, examples: int, tokens: int) -> None:
        self.consumed_examples += examples
        self.consumed_tokens += tokens
        self.pending_tokens += tokens

    def update_boundary(self, committed: bool = True) -> None:
        if committed:
            self.committed_tokens += self.pending_tokens
        self.pending_tokens = 0

    def control(self) -> Dict[str, int]:
        return {COMMITTED_TOKENS: self.committed_tokens, CONSUMED_EXAMPLES: self.consumed_examples}

    @classmethod
    def from_control(cls, control: Dict[str, int]) -> "TokenClock":
        c = cls()
        c.committed_tokens = int(control.get(COMMITTED_TOKENS, 0))
        c.consumed_tokens = c.committed_tokens
        c.consumed_examples = int(control.get(CONSUMED_EXAMPLES, 0))
        return c

    def crossed(self, before: int, point: int) -> bool:
        """Whether the committed tokens crossed ``point`` since they stood at ``before`` (cooldown / budget points)."""
        return before < point <= self.committed_tokens


@dataclass
class Interval:
    """The books of a fit's cadences.  ``add`` books a step into each; ``due(step)`` names the cadences whose period ends
    at ``step``; ``take(name)`` reads that book (the only host synchronisation), returns its summary and restarts it."""
    cadences: Dict[str, int]
    device: str = "cpu"
    books: Dict[str, Book] = field(default_factory=dict)
    started: Dict[str, float] = field(default_factory=dict)
    clock: TokenClock = field(default_factory=TokenClock)

    def __post_init__(self):
        now = time.perf_counter()
        for name in self.cadences:
            self.books[name] = Book(self.device)
            self.started[name] = now

    def add(self, loss_total, loss_mass, examples: int = 0, tokens: int = 0, flops: float = 0.0, committed: bool = True) -> None:
        for b in self.books.values():
            bookkeep(b, loss_total, loss_mass, tokens, flops)
        self.clock.dispatched(examples, tokens)
        self.clock.update_boundary(committed)

    def due(self, step: int):
        return [n for n, every in self.cadences.items() if every and step % every == 0]

    def take(self, name: str, devices: int = 1, peak_flops: Optional[float] = None) -> Dict[str, float]:
        book = self.books[name]
        r = book.read()
        now = time.perf_counter()
        elapsed = max(now - self.started[name], 1e-9)
        out = {"loss": r["loss_total"] / r["loss_mass"] if r["loss_mass"] > 0 else float("nan"),
               "steps": int(r["steps"]), "finite_steps": int(r["finite"]), "nonfinite_steps": int(r["nonfinite"]),
               "tokens_per_sec": r["tokens"] / elapsed, "step_time_ms": 1000 * elapsed / max(r["steps"], 1),
               "committed_tokens": self.clock.committed_tokens}
        if peak_flops:
            out["mfu"] = r["flops"] / elapsed / (peak_flops * devices)
        book.restart()
        self.started[name] = now
        return out
