"""Guided decoding: a ``Grammar`` restricts every step's candidates to the tokens that keep the text inside a language.

The grammar here is a deterministic finite automaton over token ids, compiled from a regular expression (Thompson
construction over characters, lifted to the vocabulary's strings by lazy subset construction, ``Grammar.from_regex``) or
given directly as transitions (``Grammar.from_transitions``).  At each step
``mask(state)`` gives the allowed next tokens, ``advance(state, token)`` the next state, and ``accepting(state)`` says whether
the text may end (the end-of-sequence token is allowed only there).  ``guided_generate`` applies it on top of greedy or
sampled decoding.

Reference: src/dew/sampling/guided.py (``Grammar``), src/dew/sampling/decoding.py (``LogitsTransform``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, FrozenSet, List, Optional, Sequence, Set, Tuple

import torch


@dataclass
class Grammar:
    transitions: Dict[int, Dict[int, int]]          # state -> token id -> next state
    start: int = 0
    accept: FrozenSet[int] = frozenset()
    vocab_size: int = 0
    _masks: Dict[int, torch.Tensor] = field(default_factory=dict, repr=False)

    @classmethod
    def from_transitions(cls, transitions, start: int, accept, vocab_size: int) -> "Grammar":
        return cls({int(s): {int(t): int(n) for t, n in row.items()} for s, row in transitions.items()}, int(start),
                   frozenset(int(a) for a in accept), vocab_size)

    @classmethod
    def from_regex(cls, pattern: str, vocabulary: Sequence[str]) -> "Grammar":
        """Compile a regular expression (literals, ``.``, classes ``[a-z0-9_]`` / ``[^...]``, ``\\d \\w \\s``, groups,
        ``|``, ``* + ?``) to a character automaton and lift it to the vocabulary: a token is allowed in a state when
        walking its characters stays inside the automaton; states that cannot reach acceptance are dropped."""
        nfa = _Nfa.parse(pattern)
        start = nfa.closure({nfa.start})
        states: Dict[FrozenSet[int], int] = {start: 0}
        order: List[FrozenSet[int]] = [start]
        transitions: Dict[int, Dict[int, int]] = {}
        accept: Set[int] = set()
        i = 0
        while i < len(order):
            cur = order[i]
            sid = states[cur]
            if nfa.accept in cur:
                accept.add(sid)
            row: Dict[int, int] = {}
            for tok, piece in enumerate(vocabulary):
                if not piece:
                    continue
                st = cur
                for ch in piece:
                    st = nfa.step(st, ch)
                    if not st:
                        break
                if not st:
                    continue
                if st not in states:
                    states[st] = len(states)
                    order.append(st)
                row[tok] = states[st]
            transitions[sid] = row
            i += 1
        # prune states from which no accepting state is reachable
        alive = set(accept)
        changed = True
        while changed:
            changed = False
            for sid, row in transitions.items():
                if sid not in alive and any(n in alive for n in row.values()):
                    alive.add(sid)
                    changed = True
        transitions = {sid: {t: n for t, n in row.items() if n in alive} for sid, row in transitions.items() if sid in alive}
        return cls(transitions, 0, frozenset(accept), len(vocabulary))

    def mask(self, state: int, device=None) -> torch.Tensor:
        key = state
        if key not in self._masks:
            m = torch.zeros(self.vocab_size, dtype=torch.bool)
            allowed = list(self.transitions.get(state, {}))
            if allowed:
                m[torch.tensor(allowed)] = True
            self._masks[key] = m
        m = self._masks[key]
        return m if device is None else m.to(device)

    def advance(self, state: int, token: int) -> int:
        return self.transitions[state][int(token)]

    def accepting(self, state: int) -> bool:
        return state in self.accept

    def dead(self, state: int) -> bool:
        return not self.transitions.get(state)


class _Nfa:
    """Thompson construction for the regular-expression subset of ``Grammar.from_regex``."""

    def __init__(self):
        self.eps: Dict[int, Set[int]] = {}
        self.edges: Dict[int, List[Tuple[object, int]]] = {}      # state -> [(predicate, next state)]
        self.n = 0
        self.start = self.accept = 0

    def new(self) -> int:
        self.n += 1
        return self.n - 1

    def add_eps(self, a: int, b: int) -> None:
        self.eps.setdefault(a, set()).add(b)

    def add_edge(self, a: int, pred, b: int) -> None:
        self.edges.setdefault(a, []).append((pred, b))

    def closure(self, states) -> FrozenSet[int]:
        stack, seen = list(states), set(states)
        while stack:
            s = stack.pop()
            for t in self.eps.get(s, ()):
                if t not in seen:
                    seen.add(t)
                    stack.append(t)
        return frozenset(seen)

    def step(self, states: FrozenSet[int], ch: str) -> FrozenSet[int]:
        nxt = {b for s in states for pred, b in self.edges.get(s, ()) if pred(ch)}
        return self.closure(nxt) if nxt else frozenset()

    # ---- parser: alternation > concatenation > repetition > atom; every fragment is a (start, end) pair
    @classmethod
    def parse(cls, pattern: str) -> "_Nfa":
        self = cls()
        self.pattern, self.pos = pattern, 0
        s, e = self._alternation()
        if self.pos != len(pattern):
            raise ValueError(f"unbalanced pattern at {self.pos}: {pattern!r}")
        self.start, self.accept = s, e
        return self

    def _peek(self) -> Optional[str]:
        return self.pattern[self.pos] if self.pos < len(self.pattern) else None

    def _alternation(self):
        frags = [self._concatenation()]
        while self._peek() == "|":
            self.pos += 1
            frags.append(self._concatenation())
        if len(frags) == 1:
            return frags[0]
        s, e = self.new(), self.new()
        for fs, fe in frags:
            self.add_eps(s, fs)
            self.add_eps(fe, e)
        return s, e

    def _concatenation(self):
        s = e = self.new()
        while self._peek() is not None and self._peek() not in "|)":
            fs, fe = self._repetition()
            self.add_eps(e, fs)
            e = fe
        return s, e

    def _repetition(self):
        fs, fe = self._atom()
        while self._peek() in ("*", "+", "?"):
            op = self.pattern[self.pos]
            self.pos += 1
            s, e = self.new(), self.new()
            self.add_eps(s, fs)
            self.add_eps(fe, e)
            if op in "*?":
                self.add_eps(s, e)
            if op in "*+":
                self.add_eps(fe, fs)
            fs, fe = s, e
        return fs, fe

    _ESCAPES = {"d": str.isdigit, "w": lambda c: c.isalnum() or c == "_", "s": str.isspace}

    def _atom(self):
        ch = self.pattern[self.pos]
        self.pos += 1
        if ch == "(":
            frag = self._alternation()
            if self._peek() != ")":
                raise ValueError("missing )")
            self.pos += 1
            return frag
        s, e = self.new(), self.new()
        if ch == ".":
            self.add_edge(s, lambda c: c != "\n", e)
        elif ch == "[":
            negate = self._peek() == "^"
            if negate:
                self.pos += 1
            items: List[object] = []
            while self._peek() != "]":
                c = self.pattern[self.pos]
                self.pos += 1
                if c == "\\":
                    c2 = self.pattern[self.pos]
                    self.pos += 1
                    items.append(self._ESCAPES.get(c2, (lambda lit: (lambda x: x == lit))(c2)))
                elif self._peek() == "-" and self.pos + 1 < len(self.pattern) and self.pattern[self.pos + 1] != "]":
                    hi = self.pattern[self.pos + 1]
                    self.pos += 2
                    items.append((lambda lo_, hi_: (lambda x: lo_ <= x <= hi_))(c, hi))
                else:
                    items.append((lambda lit: (lambda x: x == lit))(c))
            self.pos += 1
            self.add_edge(s, (lambda its, neg: (lambda x: any(p(x) for p in its) != neg))(items, negate), e)
        elif ch == "\\":
            c2 = self.pattern[self.pos]
            self.pos += 1
            self.add_edge(s, self._ESCAPES.get(c2, (lambda lit: (lambda x: x == lit))(c2)), e)
        else:
            self.add_edge(s, (lambda lit: (lambda x: x == lit))(ch), e)
        return s, e


def guided_generate(model, prompt: Sequence[int], grammar: Grammar, max_new_tokens: int, eos_token_id: Optional[int] = None,
                    temperature: float = 0.0, generator: Optional[torch.Generator] = None) -> Tuple[List[int], bool]:
    """Decode under the grammar: returns (new tokens, ended in an accepting state)."""
    dev = next(model.parameters()).device
    seq = list(prompt)
    state = grammar.start
    out: List[int] = []
    with torch.no_grad():
        for _ in range(max_new_tokens):
            logits = model(torch.tensor([seq], device=dev))[0, -1].float()
            allowed = grammar.mask(state, dev).clone()
            if eos_token_id is not None and grammar.accepting(state) and eos_token_id < allowed.numel():
                allowed[eos_token_id] = True
            if not bool(allowed.any()):
                break
            logits = logits[: allowed.numel()].masked_fill(~allowed, float("-inf"))
            if temperature > 0:
                tok = int(torch.multinomial(torch.softmax(logits / temperature, -1).cpu(), 1, generator=generator))
            else:
                tok = int(logits.argmax())
            if eos_token_id is not None and tok == eos_token_id and grammar.accepting(state):
                return out, True
            out.append(tok)
            seq.append(tok)
            state = grammar.advance(state, tok)
            if grammar.dead(state):
                break
    return out, grammar.accepting(state)
