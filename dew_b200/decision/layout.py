"""How a state and its questions become the token rows a decision model reads.

A layout places each question's instructions and each of its options at a span of tokens which a head reads back.  Three
shapes:

``marker``       one row per question, for a bidirectional backbone; a marker token stands before each option's text
                 ``[CLS] <type> question: <instructions> [SEP] [MASK] opt0 [MASK] opt1 ... [SEP] state [SEP]``
``state_first``  one row per question, for a causal backbone: the state first, each marker after its option (so the marker
                 has read the option), an answer cue last
                 ``[BOS] state [SEP] <type> question: <instructions> [SEP] opt0 [MASK] opt1 [MASK] ... [SEP] answer:``
``joint``        every question of a request in one row behind the state, each option a span of its own

With ``labels`` the options are written as lettered lines (``A. text``) and the answer is read at the cue as the backbone's
own next-token logits of the letters (``LabelReadout``).  The option texts and the instructions share ``head_max_len``
tokens (the longest texts are cut first); the state takes what is left of ``max_len`` and keeps its first tokens.  Every cut
is counted (``Encoded.cut``), and ``usage_of`` sums a request's rows into what a served answer reports.

Reference: src/dew/decision/layout.py (``SegmentLayout.marker_row`` / ``state_first_row`` / ``joint_row``, ``Specials``,
``Labels``, ``Encoded``, ``render``), src/dew/decision/task.py (``Usage``, ``usage_of``).
"""
from __future__ import annotations

import json
import string
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

from .questions import Question, kind_of

SHAPES = ("marker", "state_first", "joint")


# ------------------------------------------------------------------------------------------------ tokens
class ByteTokenizer:
    """UTF-8 bytes shifted past four special ids (pad 0, start 1, separator 2, marker 3): a vocabulary of 260 that needs no
    files.  Any object with ``encode(text) -> ids`` (a transformers tokenizer called with ``add_special_tokens=False``) fits
    where this is used."""
    pad_token_id, cls_token_id, sep_token_id, mask_token_id = 0, 1, 2, 3
    vocab_size = 260

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        return [b + 4 for b in text.encode("utf-8")]

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i - 4 for i in ids if i >= 4).decode("utf-8", errors="replace")


@dataclass(frozen=True)
class Specials:
    """The special tokens a layout places: the row's start (None for a vocabulary without one), the separator, the option
    marker and the padding id."""
    start: Optional[int]
    separator: int
    marker: int
    pad: int = 0

    @classmethod
    def of(cls, tokenizer) -> "Specials":
        def first(*names):
            for n in names:
                v = getattr(tokenizer, n, None)
                if v is not None:
                    return int(v)
            return None
        sep = first("sep_token_id", "eos_token_id")
        marker = first("mask_token_id", "unk_token_id")
        if sep is None or marker is None:
            raise ValueError("a layout needs a separator (sep / eos) and a marker (mask / unk) token in the vocabulary")
        pad = first("pad_token_id")
        return cls(first("cls_token_id", "bos_token_id"), sep, marker, 0 if pad is None else pad)


def render(state: Any) -> str:
    """A state as the text a row holds: a string as it is, anything else as compact JSON with its keys in the given order."""
    if isinstance(state, str):
        return state
    return json.dumps(state, ensure_ascii=False, separators=(", ", ": "))


def _text_of(value: Any) -> str:
    return "" if value is None else render(value)


# ------------------------------------------------------------------------------------------------ one laid-out row
@dataclass
class Encoded:
    """One row: its tokens and, per question, where the head reads it."""
    tokens: List[int]
    names: Tuple[str, ...]                      # the questions of this row, by request name
    kinds: List[int]                            # KINDS number per question
    counts: List[int]                           # options per question
    markers: List[List[int]]                    # [q][k] marker position
    spans: List[List[Tuple[int, int]]]          # [q][k] the option's text, [start, end)
    asked: List[Tuple[int, int]]                # [q] the question's instructions, [start, end)
    readout: List[int]                          # [q] the answer cue's position (the row's last token where there is none)
    token_kind: List[int]                       # per token: the kind of the question it belongs to, -1 for the state
    label_ids: Optional[List[List[int]]] = None  # [q][k] the token id of each option's letter (``labels`` layouts)
    state_tokens: int = 0                       # the state as given
    state_kept: int = 0
    cut: Dict[str, int] = field(default_factory=dict)   # tokens removed, by what was cut: state / instructions / options

    def __len__(self):
        return len(self.tokens)


@dataclass(frozen=True)
class Usage:
    """What a request cost: the tokens its rows read, how much of the state they kept (the least any row kept), and each cut
    as (rows it shortened, tokens it removed)."""
    input_tokens: int
    state_tokens: int
    state_kept: int
    cut: Mapping[str, Tuple[int, int]]

    @property
    def truncated(self) -> bool:
        return self.state_kept < self.state_tokens

    @property
    def trimmed(self) -> bool:
        return any(k != "state" for k in self.cut)


def usage_of(rows: Sequence[Encoded]) -> Usage:
    cut: Dict[str, Tuple[int, int]] = {}
    for r in rows:
        for kind, n in r.cut.items():
            if n:
                a, b = cut.get(kind, (0, 0))
                cut[kind] = (a + 1, b + n)
    return Usage(sum(len(r) for r in rows), max((r.state_tokens for r in rows), default=0),
                 min((r.state_kept for r in rows), default=0), cut)


class Refused(ValueError):
    """A request the layout cannot lay out (``reason``: unfit, options_alike, cut)."""

    def __init__(self, reason: str, message: str):
        super().__init__(message)
        self.reason = reason


# ------------------------------------------------------------------------------------------------ the layout
LETTERS = tuple(string.ascii_uppercase) + tuple(a + b for a in string.ascii_uppercase for b in string.ascii_uppercase)


@dataclass
class Layout:
    tokenizer: Any = None
    specials: Optional[Specials] = None
    shape: str = "state_first"
    max_len: int = 512
    head_max_len: int = 128
    labels: bool = False
    question_template: str = "{type} question: {instructions}"
    cue: str = "answer:"

    def __post_init__(self):
        if self.shape not in SHAPES:
            raise ValueError(f"a layout's shape is one of {SHAPES}, got {self.shape!r}")
        if self.tokenizer is None:
            self.tokenizer = ByteTokenizer()
        if self.specials is None:
            self.specials = Specials.of(self.tokenizer)
        if self.labels and self.shape == "marker":
            raise ValueError("lettered options are read at an answer cue, which the marker rows do not have")
        if self.head_max_len >= self.max_len:
            raise ValueError("head_max_len (questions and options) must leave room for the state inside max_len")
        self._pieces: Dict[str, List[int]] = {}

    # -- record (what a saved task keeps of its layout)
    def record(self) -> Dict[str, Any]:
        return {"shape": self.shape, "max_len": self.max_len, "head_max_len": self.head_max_len, "labels": self.labels,
                "question_template": self.question_template, "cue": self.cue,
                "specials": {"start": self.specials.start, "separator": self.specials.separator, "marker": self.specials.marker,
                             "pad": self.specials.pad}}

    @classmethod
    def from_record(cls, rec: Mapping[str, Any], tokenizer=None) -> "Layout":
        rec = dict(rec)
        sp = Specials(**rec.pop("specials"))
        return cls(tokenizer=tokenizer, specials=sp, **rec)

    # -- text -> ids, remembered (a corpus repeats its templates, instructions and options)
    def piece(self, text: str) -> List[int]:
        hit = self._pieces.get(text)
        if hit is None:
            ids = self.tokenizer.encode(text, add_special_tokens=False) if text else []
            ids = [i for i in ids if i != self.specials.marker]          # a caller's text never places a marker
            if len(self._pieces) >= 16384:
                self._pieces.pop(next(iter(self._pieces)))
            self._pieces[text] = hit = list(ids)
        return hit

    def _option_text(self, q: Question, k: int) -> str:
        key, desc = q.options[k], q.descriptions[k]
        body = key if desc is None else f"{key}: {_text_of(desc)}"
        return f"{LETTERS[k]}. {body}" if self.labels else body

    def _fit_head(self, instr: List[int], opts: List[List[int]], room: int, cut: Dict[str, int]):
        """Cut the option texts (longest first, a token at a time from their ends) and then the instructions until the head
        holds at most ``room`` tokens besides its fixed ones."""
        opts = [list(o) for o in opts]
        over = len(instr) + sum(len(o) for o in opts) - room
        if over <= 0:
            return instr, opts
        removed = 0
        # level the longest options down to a common ceiling
        lengths = sorted((len(o) for o in opts), reverse=True)
        ceiling = lengths[0] if lengths else 0
        while over > 0 and ceiling > 1:
            above = sum(max(0, len(o) - (ceiling - 1)) for o in opts)
            take = min(over, above)
            if take == 0:
                break
            for o in opts:
                while take and len(o) > ceiling - 1:
                    o.pop()
                    take -= 1
                    over -= 1
                    removed += 1
            ceiling -= 1
        if removed:
            cut["options"] = cut.get("options", 0) + removed
        if over > 0:
            keep = max(1, len(instr) - over)
            cut["instructions"] = cut.get("instructions", 0) + len(instr) - keep
            over -= len(instr) - keep
            instr = instr[:keep]
        if over > 0:
            raise Refused("unfit", f"the questions and options do not fit head_max_len={self.head_max_len} tokens even when cut")
        return instr, opts

    def _question_block(self, q: Question, at: int, cut: Dict[str, int], room: int):
        """Tokens of one question and where its parts sit, starting at position ``at``."""
        sp = self.specials
        instr = self.piece(self.question_template.format(type=q.kind, instructions=_text_of(q.instructions)))
        opts = [self.piece(self._option_text(q, k)) for k in range(len(q.options))]
        if len({tuple(o) for o in opts}) != len(opts):
            raise Refused("options_alike", "two options of a question read as the same tokens")
        fixed = 2 + len(opts)                                            # two separators and one marker per option
        instr, opts = self._fit_head(instr, opts, room - fixed, cut)
        if len({tuple(o) for o in opts}) != len(opts):
            raise Refused("options_alike", "two options of a question read as the same tokens once cut to the head's room")
        toks: List[int] = []
        asked = (at, at + len(instr))
        toks += instr + [sp.separator]
        markers, spans = [], []
        for o in opts:
            if self.shape == "marker":
                markers.append(at + len(toks))
                toks.append(sp.marker)
                spans.append((at + len(toks), at + len(toks) + len(o)))
                toks += o
            else:
                spans.append((at + len(toks), at + len(toks) + len(o)))
                toks += o
                markers.append(at + len(toks))
                toks.append(sp.marker)
        toks.append(sp.separator)
        return toks, asked, markers, spans

    def rows(self, state: Any, questions: Mapping[str, Question]) -> List[Encoded]:
        """The request's rows: one per question (``marker``, ``state_first``) or one for all of them (``joint``)."""
        if not questions:
            raise Refused("unfit", "a request needs at least one question")
        if self.shape == "joint":
            return [self._row(state, tuple(questions.items()))]
        return [self._row(state, ((name, q),)) for name, q in questions.items()]

    def _row(self, state: Any, asked_qs: Sequence[Tuple[str, Question]]) -> Encoded:
        sp = self.specials
        state_ids = self.piece(render(state))
        cut: Dict[str, int] = {}
        start = [] if sp.start is None else [sp.start]
        cue = self.piece(self.cue) if self.shape != "marker" else []
        room_each = self.head_max_len // len(asked_qs) if self.shape == "joint" else self.head_max_len
        # lay the question blocks out at offset 0 first to know their sizes, then place them
        blocks = [self._question_block(q, 0, cut, room_each) for _, q in asked_qs]
        head_len = sum(len(b[0]) for b in blocks) + (len(cue) * len(asked_qs) if self.shape != "marker" else 0)
        room_state = self.max_len - len(start) - head_len - 1
        if room_state < 1 and state_ids:
            raise Refused("unfit", f"the questions leave no room for the state inside max_len={self.max_len}")
        kept = state_ids[:max(0, room_state)]
        if len(kept) < len(state_ids):
            cut["state"] = len(state_ids) - len(kept)
        tokens: List[int] = list(start)
        token_kind: List[int] = [-1] * len(tokens)
        out = Encoded(tokens, tuple(n for n, _ in asked_qs), [], [], [], [], [], [], token_kind,
                      [] if self.labels else None, len(state_ids), len(kept), cut)

        def place(qi: int):
            name, q = asked_qs[qi]
            toks, asked, markers, spans = blocks[qi]
            at = len(tokens)
            tokens.extend(toks)
            kind = kind_of(q)
            token_kind.extend([kind] * len(toks))
            out.kinds.append(kind)
            out.counts.append(len(q.options))
            out.asked.append((asked[0] + at, asked[1] + at))
            out.markers.append([m + at for m in markers])
            out.spans.append([(a + at, b + at) for a, b in spans])
            if self.shape != "marker":
                tokens.extend(cue)
                token_kind.extend([kind] * len(cue))
                out.readout.append(len(tokens) - 1)
            if self.labels:
                ids = []
                for k in range(len(q.options)):
                    letter = self.piece(" " + LETTERS[k]) or self.piece(LETTERS[k])
                    ids.append(letter[-1])
                out.label_ids.append(ids)

        if self.shape == "marker":
            place(0)
            tokens.extend(kept + [sp.separator])
            token_kind.extend([-1] * (len(kept) + 1))
            out.readout.append(0)
            if len(asked_qs) == 1:
                out.token_kind[:] = [out.kinds[0]] * len(tokens)          # the row's one type, added to every state
        else:
            tokens.extend(kept + [sp.separator])
            token_kind.extend([-1] * (len(kept) + 1))
            for qi in range(len(asked_qs)):
                place(qi)
            if self.shape == "state_first":
                out.token_kind[:] = [out.kinds[0]] * len(tokens)
        if len(tokens) > self.max_len:
            raise Refused("unfit", f"a row of {len(tokens)} tokens does not fit max_len={self.max_len}")
        return out

    # -- what a batch must hold of a corpus
    def bounds(self, questions_per_request: int, options: int) -> Tuple[int, int]:
        """(question slots per row, option slots per question)."""
        return (questions_per_request if self.shape == "joint" else 1), options
