"""Decision models: one forward pass answers typed questions about a state.

A request is a state (text, or any JSON) and named questions, each a ``Noul`` (yes / no), a ``Choice`` among named options or a
``Score`` over ordered levels.  A ``Layout`` writes the questions out with the state as token rows (one row per question with a
marker per option, state-first rows for a causal backbone, or every question of a request in one joint row), rows are packed
first-fit into windows, a backbone reads them, a head scores every option (``DecisionHead`` at the markers, ``JointSchemaHead``
over pooled option spans, ``LabelReadout`` / ``SlotReadout`` at an answer cue), and the answer is a distribution over exactly the
options each question names.  ``DecisionObjective`` trains on proper scoring rules (with label smoothing and a consistency term
over grouped questions), ``Calibration`` (temperatures, binning, abstention per bucket) turns raw logits into reported answers,
and ``Decide`` answers requests inside a token budget, plays wide choices as tournaments and speaks the JSON wire form.

Reference: src/dew/decision/ (questions, layout, inputs, head, model, data, objective, scoring, metrics, calibration, task).
"""
from .calibration import Abstention, Binning, Calibration, Scored, Temperatures, bucket
from .data import Example, Group, GroupedExamples, ParseTable, decisions, mixture
from .head import DecisionHead, Head, JointSchemaHead, LabelReadout, SlotReadout
from .inputs import DecisionInputs, collate, first_fit
from .layout import ByteTokenizer, Encoded, Layout, Refused, Specials, Usage, render, usage_of
from .metrics import AURC, ECE, Accuracy, Decisions, MacroF1, ScoredQuestions, default_metrics, measure
from .model import BidirectionalBackbone, DecisionModel
from .objective import DecisionObjective
from .questions import (KINDS, Answer, Choice, ChoiceAnswer, Confidence, EntropyConfidence, JevConfidence, Noul, NoulAnswer, Question,
                        Score, ScoreAnswer, TopProbability, kind_of)
from .scoring import Brier, Combined, LogLoss, RankedProbability, ScoringRule, Spherical
from .task import TASK_FILE, Budget, Decide, Finalists, Knockout, Request

__all__ = [n for n in dir() if not n.startswith("_")]
