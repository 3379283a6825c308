"""``Decide``: a decision model answering requests, as typed answers and in the JSON request / response form.

``decide(state, questions)`` returns one answer per question with probabilities over exactly the question's options;
``decide(requests)`` answers many requests, their rows packed first-fit into passes that each stay inside the ``Budget`` (so
every pass takes one of a few shapes, and a CUDA graph or a warmed allocator serves all of them).  A choice too wide for one
row is played as a tournament: ``Knockout`` (group winners go on, round after round; the answer covers the last round's
options) or ``Finalists`` (the best ``keep`` of each group go to one final; the answer covers every option, the finalists
sharing ``1 - residual`` as the final gave it and the rest ``residual`` in proportion to their group round).  ``calibrated``
fits the calibration on held-out examples; ``systemone`` takes and returns the wire form:

    {"state": ..., "questions": {name: {"type", "instructions", "criteria"}}}
    -> {"model", "answers": {name: {"type", ...}}, "usage": {"input_tokens", "output_tokens"}}

Reference: src/dew/decision/task.py (``Budget``, ``Knockout``, ``Finalists``, ``Usage``, ``Decide.decide`` / ``systemone`` /
``calibrated`` / ``save`` / ``from_run``, the first-fit ``PassPlan``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .calibration import Calibration, Scored
from .data import Example
from .inputs import collate, first_fit
from .layout import Encoded, Layout, Refused, Usage, usage_of
from .model import DecisionModel
from .questions import Answer, Choice, ChoiceAnswer, Confidence, JevConfidence, NoulAnswer, Question, ScoreAnswer

TASK_FILE = "decide.json"


@dataclass(frozen=True)
class Budget:
    """How much one forward pass may hold: at most ``tokens`` tokens in at most ``rows`` windows; ``lengths`` are the window
    lengths a pass may take (the shortest that holds the pass's longest row is used)."""
    tokens: int = 16384
    rows: int = 256
    lengths: Tuple[int, ...] = (128, 256, 512, 1024, 2048)
    options: Optional[int] = None

    def windows(self, length: int) -> int:
        return max(1, min(self.rows, self.tokens // length))


@dataclass(frozen=True)
class Knockout:
    group: int = 16

    def __post_init__(self):
        if self.group < 2:
            raise ValueError("a tournament groups at least two options")


@dataclass(frozen=True)
class Finalists:
    group: int = 25
    keep: int = 3
    final: int = 26
    residual: float = 1e-3

    def __post_init__(self):
        if not (self.group >= 2 and 1 <= self.keep <= self.group and self.final >= 2 and 0 <= self.residual < 1):
            raise ValueError("finalists need 2 <= group, 1 <= keep <= group, 2 <= final and 0 <= residual < 1")


def near_equal(options: Sequence[str], group: int) -> List[List[str]]:
    """Consecutive groups of at most ``group``, as equal as possible, the first ones one longer."""
    parts = -(-len(options) // group)
    size, extra = divmod(len(options), parts)
    out, at = [], 0
    for p in range(parts):
        n = size + (p < extra)
        out.append(list(options[at:at + n]))
        at += n
    return out


def knocked_out(final: Mapping[str, float], first: Mapping[str, float], residual: float) -> Dict[str, float]:
    rest = [o for o in first if o not in final]
    mass = sum(first[o] for o in rest)
    spread = {o: float(v) * (1 - residual) for o, v in final.items()}
    for o in rest:
        spread[o] = residual * first[o] / mass if mass else residual / len(rest)
    total = sum(spread.values())
    return {o: v / total for o, v in spread.items()}


@dataclass
class Request:
    state: Any
    questions: Mapping[str, Question]


class Decide:
    def __init__(self, model: DecisionModel, layout: Layout, *, calibration: Optional[Calibration] = None,
                 confidence: Optional[Confidence] = None, budget: Budget = Budget(), tournament: Union[Knockout, Finalists, None] = None,
                 name: str = "dew-b200-decision", device=None):
        self.model, self.layout = model, layout
        self.calibration = calibration or Calibration()
        self.confidence = confidence or JevConfidence()
        self.budget, self.tournament, self.name = budget, tournament, name
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.passes: List[Tuple[int, int, int]] = []          # (length, windows, real tokens) of every pass run

    # ------------------------------------------------------------------ scoring rows
    @torch.no_grad()
    def logits(self, rows: Sequence[Encoded]) -> List[np.ndarray]:
        """Raw ``[Q, K]`` logits of every row (its questions in row order, its options in question order), scored in passes
        inside the budget."""
        out: List[Optional[np.ndarray]] = [None] * len(rows)
        pending = list(range(len(rows)))
        was_training = self.model.training
        self.model.eval()
        try:
            while pending:
                longest = len(rows[pending[0]])
                # a pass grows row by row while a length holds it: take the shortest declared length that fits the first row,
                # then first-fit the rest into that length's windows
                length = next((l for l in self.budget.lengths if l >= longest), None)
                if length is None:
                    raise Refused("unfit", f"a row of {longest} tokens is past the longest pass length {self.budget.lengths[-1]}")
                fits = [i for i in pending if len(rows[i]) <= length]
                sub = [rows[i] for i in fits]
                windows, leftover = first_fit(sub, length, self.budget.windows(length))
                taken = [fits[j] for w in windows for j in w]
                Q = max(sum(len(sub[j].names) for j in w) for w in windows)
                K = self.budget.options or max(max(sub[j].counts) for w in windows for j in w)
                K = 1 << (K - 1).bit_length() if self.budget.options is None else K
                inputs, where = collate(sub, windows, length, Q, K, self.layout.specials.pad)
                lg = self.model(inputs.to(self.device)).float().cpu().numpy()
                self.passes.append((length, len(windows), sum(len(sub[j]) for w in windows for j in w)))
                for j, slots in enumerate(where):
                    if slots:
                        out[fits[j]] = np.stack([lg[b, q, : max(sub[j].counts)] for b, q in slots])
                done = set(taken)
                pending = [i for i in pending if i not in done]
        finally:
            self.model.train(was_training)
        return out            # type: ignore[return-value]

    def real_token_share(self) -> float:
        """The share of the computed tokens that were rows' real tokens, over every pass so far."""
        computed = sum(l * w for l, w, _ in self.passes)
        return sum(r for _, _, r in self.passes) / computed if computed else 1.0

    # ------------------------------------------------------------------ answers
    def _answer(self, q: Question, logits: np.ndarray) -> Answer:
        p, _, abstained = self.calibration.apply(q, logits[: len(q.options)])
        return q.answer(p, self.confidence, abstained)

    def _rows_of(self, state: Any, questions: Mapping[str, Question]) -> Tuple[List[Encoded], Dict[str, Question]]:
        narrow = {n: q for n, q in questions.items() if not self._wide(q)}
        return (self.layout.rows(state, narrow) if narrow else []), narrow

    def _wide(self, q: Question) -> bool:
        t = self.tournament
        if t is None or not isinstance(q, Choice):
            return False
        return len(q.options) > (t.group if isinstance(t, Knockout) else t.final)

    def decide(self, state_or_requests, questions: Optional[Mapping[str, Question]] = None):
        if questions is not None:
            return self.decide([Request(state_or_requests, questions)])[0]
        requests = [r if isinstance(r, Request) else Request(r["state"], r["questions"]) for r in state_or_requests]
        rows: List[Encoded] = []
        owner: List[Tuple[int, Encoded]] = []
        for ri, r in enumerate(requests):
            laid, _ = self._rows_of(r.state, r.questions)
            rows += laid
            owner += [(ri, e) for e in laid]
        scored = self.logits(rows) if rows else []
        answers: List[Dict[str, Answer]] = [dict() for _ in requests]
        for (ri, e), lg in zip(owner, scored):
            for qi, name in enumerate(e.names):
                answers[ri][name] = self._answer(requests[ri].questions[name], lg[qi])
        for ri, r in enumerate(requests):
            for name, q in r.questions.items():
                if self._wide(q):
                    answers[ri][name] = self._tournament(r.state, q)
            answers[ri] = {n: answers[ri][n] for n in r.questions}          # the request's own order
        return answers

    def _round(self, state: Any, q: Choice, groups: Sequence[Sequence[str]]) -> List[Dict[str, float]]:
        """Each group of options asked as a question of its own over ``state``: per group, option -> probability."""
        asked = {f"g{i}": q.restricted(g) for i, g in enumerate(groups)}
        rows = []
        for name, sub in asked.items():
            rows += self.layout.rows(state, {name: sub})
        out = []
        for (name, sub), lg in zip(asked.items(), self.logits(rows)):
            p, _, _ = self.calibration.apply(sub, lg[0][: len(sub.options)])
            out.append(dict(zip(sub.options, p.tolist())))
        return out

    def _tournament(self, state: Any, q: Choice) -> ChoiceAnswer:
        t = self.tournament
        if isinstance(t, Knockout):
            options = list(q.options)
            while len(options) > t.group:
                rounds = self._round(state, q, near_equal(options, t.group))
                options = [max(r, key=r.get) for r in rounds]
            final = self._round(state, q, [options])[0]
            sub = q.restricted(options)
            return sub.answer(np.array([final[o] for o in options]), self.confidence)
        groups = near_equal(list(q.options), t.group)
        first_rounds = self._round(state, q, groups)
        first: Dict[str, float] = {}
        finalists: List[Tuple[str, float]] = []
        for r in first_rounds:
            first.update(r)
            finalists += sorted(r.items(), key=lambda kv: -kv[1])[: t.keep]
        if len(finalists) > t.final:
            keep = set(o for o, _ in sorted(finalists, key=lambda kv: -kv[1])[: t.final])
            finalists = [f for f in finalists if f[0] in keep]
        names = [o for o, _ in finalists]
        final = self._round(state, q, [names])[0]
        spread = knocked_out(final, first, t.residual)
        return q.answer(np.array([spread[o] for o in q.options]), self.confidence)

    # ------------------------------------------------------------------ calibration
    def scored(self, examples: Sequence[Example]) -> List[Scored]:
        rows, golds = [], []
        for ex in examples:
            for r in self.layout.rows(ex.state, ex.questions):
                rows.append(r)
                golds.append([(ex.questions[n], ex.distribution(n)) for n in r.names])
        out = []
        for lg, gs in zip(self.logits(rows), golds):
            for qi, (q, gold) in enumerate(gs):
                if gold is not None:
                    out.append(Scored.of(q, lg[qi][: len(q.options)], gold))
        return out

    def calibrated(self, examples: Sequence[Example], bins: Optional[int] = 10, target_error: Optional[float] = None, least: int = 20) -> "Decide":
        cal = Calibration.fit(self.scored(examples), bins, target_error, least)
        return Decide(self.model, self.layout, calibration=cal, confidence=self.confidence, budget=self.budget,
                      tournament=self.tournament, name=self.name, device=self.device)

    # ------------------------------------------------------------------ the wire form
    def systemone(self, request, *, details: bool = False, strict: bool = False, whole: bool = False):
        if isinstance(request, Mapping):
            out = self._systemone([request], details, strict, whole)[0]
            if isinstance(out, ValueError):
                raise out
            return out
        return self._systemone(list(request), details, strict, whole)

    def _read_wire(self, request: Mapping[str, Any]) -> Request:
        extra = set(request) - {"state", "questions", "model"}
        if extra:
            raise ValueError(f"a request holds state, questions and model, not {sorted(extra)}")
        if "state" not in request:
            raise ValueError("a request needs a state")
        qs = request.get("questions")
        if not isinstance(qs, Mapping) or not qs:
            raise ValueError("a request needs at least one question")
        return Request(request["state"], {n: Question.from_wire(w) for n, w in qs.items()})

    def _systemone(self, bodies, details: bool, strict: bool, whole: bool):
        if strict and details:
            raise ValueError("strict answers hold the wire's own fields alone, so they carry no details")
        admitted: Dict[int, Tuple[Request, List[Encoded]]] = {}
        out: Dict[int, Any] = {}
        for i, body in enumerate(bodies):
            try:
                r = self._read_wire(body)
                rows, _ = self._rows_of(r.state, r.questions)
                usage = usage_of(rows)
                if whole and (usage.truncated or usage.trimmed):
                    what = "state" if usage.truncated else "instructions or options"
                    raise Refused("cut", f"the request does not fit the maximum context length, max_len={self.layout.max_len} tokens, "
                                         f"without cutting its {what}")
                admitted[i] = (r, rows)
            except ValueError as refused:
                out[i] = refused
        order = list(admitted)
        all_rows = [e for i in order for e in admitted[i][1]]
        scored = self.logits(all_rows) if all_rows else []
        at = 0
        gated = self.calibration.abstention is not None
        for i in order:
            r, rows = admitted[i]
            answers: Dict[str, Answer] = {}
            for e in rows:
                for qi, name in enumerate(e.names):
                    answers[name] = self._answer(r.questions[name], scored[at][qi])
                at += 1
            for name, q in r.questions.items():
                if self._wide(q):
                    answers[name] = self._tournament(r.state, q)
            usage = usage_of(rows)
            reported: Dict[str, Any] = {"input_tokens": usage.input_tokens, "output_tokens": 0}
            if details:
                reported.update(state_tokens=usage.state_tokens, state_kept=usage.state_kept, truncated=usage.truncated,
                                cut={k: {"rows": a, "removed": b, "unit": "tokens"} for k, (a, b) in usage.cut.items()})
            out[i] = {"model": self.name,
                      "answers": {n: _wire(r.questions[n], answers[n], details=details, gated=gated) for n in r.questions},
                      "usage": reported}
        return [out[i] for i in range(len(bodies))]

    # ------------------------------------------------------------------ as a served task
    def scoring(self, *, details: bool = False, strict: bool = False, whole: bool = False) -> "WireScoring":
        """This task as a scoring task of wire bodies for ``inference.scoring.ScoringServer``: bodies submitted from many threads
        are laid out as they arrive and their rows scored together, a pass at a time."""
        if strict and details:
            raise ValueError("strict answers hold the wire's own fields alone, so they carry no details")
        return WireScoring(self, details, strict, whole)

    # ------------------------------------------------------------------ saving
    def save(self, directory: str, weights: bool = True) -> str:
        os.makedirs(directory, exist_ok=True)
        t = self.tournament
        rec = {"name": self.name, "layout": self.layout.record(), "model": self.model.record(), "calibration": self.calibration.record(),
               "budget": {"tokens": self.budget.tokens, "rows": self.budget.rows, "lengths": list(self.budget.lengths), "options": self.budget.options},
               "tournament": None if t is None else {"rule": type(t).__name__, **t.__dict__},
               "confidence": type(self.confidence).__name__}
        path = os.path.join(directory, TASK_FILE)
        with open(path + ".tmp", "w") as f:
            json.dump(rec, f, indent=1)
        os.replace(path + ".tmp", path)
        if weights:
            from safetensors.torch import save_file
            save_file({k: v.detach().cpu().contiguous() for k, v in self.model.state_dict().items()}, os.path.join(directory, "decide.safetensors"))
        return path

    @classmethod
    def load(cls, directory: str, model: DecisionModel, tokenizer=None, device=None) -> "Decide":
        """Read a saved task back around ``model`` (built by the caller as the record's ``model`` entry describes)."""
        from . import questions as Q
        with open(os.path.join(directory, TASK_FILE)) as f:
            rec = json.load(f)
        weights = os.path.join(directory, "decide.safetensors")
        if os.path.exists(weights):
            from safetensors.torch import load_file
            model.load_state_dict(load_file(weights))
        b = rec["budget"]
        t = rec.get("tournament")
        tour = None
        if t is not None:
            t = dict(t)
            tour = {"Knockout": Knockout, "Finalists": Finalists}[t.pop("rule")](**t)
        return cls(model, Layout.from_record(rec["layout"], tokenizer), calibration=Calibration.from_record(rec["calibration"]),
                   confidence=getattr(Q, rec.get("confidence", "JevConfidence"))(),
                   budget=Budget(b["tokens"], b["rows"], tuple(b["lengths"]), b.get("options")), tournament=tour, name=rec["name"], device=device)


class WireScoring:
    """``Decide`` behind a ``ScoringServer``: ``admit`` parses and lays out a body (refusing what the wire form refuses, a body that
    would have to be cut under ``whole`` included), ``forward`` scores rows inside the task's budget, ``answer`` builds the
    response body.  Wide choices (tournaments) are played at answer time, outside the shared passes."""

    def __init__(self, decide: Decide, details: bool, strict: bool, whole: bool):
        self.decide, self.details, self.strict, self.whole = decide, details, strict, whole
        self.admitted = 0
        self.refusals: Dict[str, int] = {}

    def admit(self, request):
        from ..inference.scoring import ScoringRequest
        d = self.decide
        try:
            r = d._read_wire(request)
            rows, _ = d._rows_of(r.state, r.questions)
            usage = usage_of(rows)
            if self.whole and (usage.truncated or usage.trimmed):
                what = "state" if usage.truncated else "instructions or options"
                raise Refused("cut", f"the request does not fit the maximum context length, max_len={d.layout.max_len} tokens, "
                                     f"without cutting its {what}")
        except ValueError as refused:
            reason = getattr(refused, "reason", "malformed")
            self.refusals[reason] = self.refusals.get(reason, 0) + 1
            raise
        self.admitted += 1
        return ScoringRequest(tuple(rows), (r, usage))

    def forward(self, rows):
        return self.decide.logits(list(rows))

    def answer(self, payload, outputs):
        d = self.decide
        r, usage = payload
        answers: Dict[str, Answer] = {}
        narrow = [n for n, q in r.questions.items() if not d._wide(q)]
        at = 0
        if d.layout.shape == "joint":
            for qi, name in enumerate(narrow):
                answers[name] = d._answer(r.questions[name], outputs[0][qi])
        else:
            for name in narrow:
                answers[name] = d._answer(r.questions[name], outputs[at][0])
                at += 1
        for name, q in r.questions.items():
            if d._wide(q):
                answers[name] = d._tournament(r.state, q)
        reported: Dict[str, Any] = {"input_tokens": usage.input_tokens, "output_tokens": 0}
        if self.details:
            reported.update(state_tokens=usage.state_tokens, state_kept=usage.state_kept, truncated=usage.truncated,
                            cut={k: {"rows": a, "removed": b, "unit": "tokens"} for k, (a, b) in usage.cut.items()})
        gated = d.calibration.abstention is not None
        return {"model": d.name, "answers": {n: _wire(r.questions[n], answers[n], details=self.details, gated=gated) for n in r.questions},
                "usage": reported}

    def metrics(self):
        return {"admitted": float(self.admitted), "real_token_share": self.decide.real_token_share(),
                **{f"refused/{k}": float(v) for k, v in self.refusals.items()}}


def _wire(q: Question, a: Answer, *, details: bool, gated: bool) -> Dict[str, Any]:
    probs = [round(float(v), 4) for v in a.probabilities]
    wire: Dict[str, Any] = {"type": q.kind}
    if isinstance(a, NoulAnswer):
        wire["noul"] = round(a.noul, 4)
        if details:
            wire["confidence"] = round(a.confidence, 4)
    elif isinstance(a, ChoiceAnswer):
        wire.update(choice=a.choice, probabilities=dict(zip(a.options, probs)), confidence=round(a.confidence, 4))
    else:
        wire.update(score=round(a.score, 4), legend=list(a.legend), probabilities=probs, confidence=round(a.confidence, 4))
    if details and gated:
        wire["abstained"] = bool(a.abstained)
    return wire
