"""Labelled requests: what a decision model trains and calibrates on.

``Example``          one state, its named questions and the right answer to some of them (an option's key or index), or a target
                     distribution where the gold is soft (a teacher's, a panel's); a question with neither is asked but not scored
``Group``            questions of one example that ask the same thing (negated, paraphrased, options re-ordered): each member
                     maps its option keys onto canonical keys the members share, so a consistency term can hold their answers
                     to one distribution
``GroupedExamples``  several examples whose rows train together, with groups across them (members keyed ``"<index>.<question>"``)
``ParseTable``       a flat table's row (``text``, ``label`` columns) as a one-question example
``decisions``        rows -> examples, inferring a table's options from its labels where none are given
``mixture``          examples drawn from several sources in given proportions, reproducibly

Reference: src/dew/decision/data.py (``Example``, ``Group``, ``GroupedExamples``, ``ParseTable``, ``decisions``, ``mixture``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, Iterator, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np

from .questions import Choice, Noul, Question, Score


@dataclass(frozen=True)
class Group:
    name: str
    members: Mapping[str, Mapping[str, str]]       # question name -> {option key -> canonical key}

    def canonical(self) -> Tuple[str, ...]:
        keys: List[str] = []
        for m in self.members.values():
            for c in m.values():
                if c not in keys:
                    keys.append(c)
        return tuple(keys)


def _check_groups(groups: Sequence[Group], question_of) -> None:
    seen = set()
    for g in groups:
        if len(g.members) < 2:
            raise ValueError(f"group {g.name!r} needs two members or more: one question is consistent with itself")
        canon = None
        for member, mapping in g.members.items():
            if member in seen:
                raise ValueError(f"question {member!r} stands in two groups")
            seen.add(member)
            q = question_of(member)
            if set(mapping) != set(q.options):
                raise ValueError(f"group {g.name!r} must map every option of {member!r}: {q.options}, got {sorted(mapping)}")
            if len(set(mapping.values())) != len(mapping):
                raise ValueError(f"group {g.name!r} maps two options of {member!r} onto one canonical key")
            keys = set(mapping.values())
            if canon is not None and keys != canon:
                raise ValueError(f"the members of group {g.name!r} do not share their canonical keys")
            canon = keys


@dataclass
class Example:
    state: Any
    questions: Mapping[str, Question]
    answers: Mapping[str, Any] = field(default_factory=dict)
    targets: Mapping[str, Any] = field(default_factory=dict)
    groups: Sequence[Group] = ()
    weight: float = 1.0

    def __post_init__(self):
        for name in list(self.answers) + list(self.targets):
            if name not in self.questions:
                raise ValueError(f"an answer to {name!r}, which the example does not ask ({sorted(self.questions)})")
        both = set(self.answers) & set(self.targets)
        if both:
            raise ValueError(f"{sorted(both)} have both an answer and a target distribution: give one")
        for name, label in self.answers.items():
            self.questions[name].index(label)
        if self.groups:
            _check_groups(self.groups, lambda m: self.questions[m])

    def distribution(self, name: str) -> Optional[np.ndarray]:
        """The gold distribution over ``name``'s options, or None where it is asked but not scored."""
        q = self.questions[name]
        n = len(q.options)
        if name in self.answers:
            t = np.zeros(n)
            t[q.index(self.answers[name])] = 1.0
            return t
        if name in self.targets:
            raw = self.targets[name]
            if isinstance(raw, Mapping):
                extra = set(raw) - set(q.options)
                if extra:
                    raise ValueError(f"target keys {sorted(extra)} are none of {name!r}'s options")
                t = np.array([float(raw.get(o, 0.0)) for o in q.options])
            else:
                t = np.asarray(raw, np.float64)
                if t.shape != (n,):
                    raise ValueError(f"a target for {name!r} needs {n} probabilities, got shape {t.shape}")
            if np.any(t < 0) or not t.sum() > 0:
                raise ValueError(f"a target distribution is non-negative with positive mass ({name!r})")
            return t / t.sum()
        return None

    @classmethod
    def of(cls, row: Mapping[str, Any]) -> "Example":
        """A row of an example's fields: ``state``, ``questions`` (wire form or ``Question``), ``answers``, ``targets``, ``groups``."""
        qs = {n: (q if isinstance(q, Question) else Question.from_wire(q)) for n, q in row["questions"].items()}
        groups = [g if isinstance(g, Group) else Group(n, g) for n, g in (row.get("groups") or {}).items()] \
            if isinstance(row.get("groups"), Mapping) else list(row.get("groups") or ())
        return cls(row["state"], qs, dict(row.get("answers") or {}), dict(row.get("targets") or {}), groups, float(row.get("weight", 1.0)))


@dataclass
class GroupedExamples:
    examples: Sequence[Example]
    groups: Sequence[Group] = ()

    def __post_init__(self):
        def q_of(member: str) -> Question:
            idx, _, name = member.partition(".")
            try:
                return self.examples[int(idx)].questions[name]
            except (ValueError, IndexError, KeyError):
                raise ValueError(f"a grouped member is '<example index>.<question>', got {member!r}") from None
        if self.groups:
            _check_groups(self.groups, q_of)


@dataclass
class ParseTable:
    """A flat row -> a one-question ``Example``.  The label names its option by key, or by index where it is an int; with
    ``by_value`` the options are the label column's own values and every label names its option by value."""
    question: Question
    text: str = "text"
    label: str = "label"
    name: str = "label"
    by_value: bool = False

    def __call__(self, row: Mapping[str, Any]) -> Example:
        if isinstance(row, Example):
            return row
        lab = row.get(self.label)
        answers = {}
        if lab is not None:
            answers[self.name] = str(lab) if self.by_value else (int(lab) if isinstance(lab, (int, np.integer)) and not isinstance(lab, bool) else lab)
        return Example(row[self.text], {self.name: self.question}, answers, weight=float(row.get("weight", 1.0)))


def decisions(rows: Iterable[Mapping[str, Any]], question: Optional[Question] = None, *, instructions: str = "Which class is this?",
              options: Optional[Sequence[str]] = None, text: str = "text", label: str = "label", name: str = "label") -> List[Example]:
    """Rows as examples.  Rows that hold ``questions`` are parsed as examples (``Example.of``); a flat table's ``text`` / ``label``
    columns become one question over ``options`` (inferred, sorted, from the labels where none are given)."""
    rows = list(rows)
    if not rows:
        return []
    if isinstance(rows[0], Example) or "questions" in rows[0]:
        return [r if isinstance(r, Example) else Example.of(r) for r in rows]
    by_value = False
    if question is None:
        if options is None:
            values = sorted({r[label] for r in rows if r.get(label) is not None}, key=str)
            options = [str(v) for v in values]
            by_value = True
        question = Noul(instructions) if list(options) == ["false", "true"] else Choice(instructions, list(options))
    parse = ParseTable(question, text, label, name, by_value=by_value)
    return [parse(r) for r in rows]


def mixture(sources: Mapping[str, Sequence[Example]], weights: Mapping[str, float], count: int, seed: int = 0) -> Iterator[Example]:
    """``count`` examples, each from source s with probability ``weights[s]``, walking every source in order (wrapping)."""
    names = list(sources)
    p = np.array([float(weights[n]) for n in names])
    if np.any(p < 0) or p.sum() <= 0:
        raise ValueError("a mixture's weights are non-negative with positive mass")
    rng = np.random.default_rng(seed)
    at = {n: 0 for n in names}
    for pick in rng.choice(len(names), size=count, p=p / p.sum()):
        n = names[int(pick)]
        src = sources[n]
        yield src[at[n] % len(src)]
        at[n] += 1
